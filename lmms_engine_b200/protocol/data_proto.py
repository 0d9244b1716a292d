"""Record schemas for chat-style SFT and preference data.

OpenAI-style ``messages`` whose ``content`` items are text / image_url / audio_url /
video_url parts (reference: src/lmms_engine/protocol/data_proto.py:6-67).
"""
from typing import List, Literal, Optional, Union

from pydantic import BaseModel


class UrlRef(BaseModel):
    url: str


class VideoUrlRef(BaseModel):
    url: str
    video_start: Optional[float] = None
    video_end: Optional[float] = None


class SFTChatDataText(BaseModel):
    type: Literal["text"]
    text: str
    precomputed_tokens: Optional[int] = None


class SFTChatDataImage(BaseModel):
    type: Literal["image_url"]
    image_url: UrlRef
    precomputed_tokens: Optional[int] = None


class SFTChatDataAudio(BaseModel):
    type: Literal["audio_url"]
    audio_url: UrlRef
    precomputed_tokens: Optional[int] = None


class SFTChatDataVideo(BaseModel):
    type: Literal["video_url"]
    video_url: VideoUrlRef
    precomputed_tokens: Optional[int] = None


SFTChatDataContent = Union[SFTChatDataText, SFTChatDataImage, SFTChatDataAudio, SFTChatDataVideo]


class SFTChatDataMessages(BaseModel):
    role: Literal["user", "system", "assistant"]
    content: List[SFTChatDataContent]


class SFTChatData(BaseModel):
    messages: List[SFTChatDataMessages]
    id: Optional[Union[int, str]] = None


class PreferenceData(BaseModel):
    id: Optional[Union[int, str]] = None
    prompt: List[SFTChatDataMessages]
    chosen: List[SFTChatDataMessages]
    rejected: List[SFTChatDataMessages]
