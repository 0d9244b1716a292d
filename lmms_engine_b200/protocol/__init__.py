from .args import Args
from .data_proto import PreferenceData, SFTChatData, SFTChatDataContent, SFTChatDataMessages
from .lmms_proto import Processable, Runnable

__all__ = ["Args", "SFTChatData", "SFTChatDataMessages", "SFTChatDataContent", "PreferenceData", "Runnable", "Processable"]
