"""Media loading for datasets: images (PIL), audio (soundfile / librosa when installed, wav
via the standard library otherwise) and video with the backends ``decord | qwen_vl_utils |
qwen_omni_utils | lmms_video_utils`` when importable and an OpenCV reader as the built-in
fallback; ``fps`` and ``frame_num`` sampling.  Reference:
src/lmms_engine/datasets/multimodal_mixin.py:40-366."""
from __future__ import annotations

import io
import os
import wave
from typing import Any, List, Optional, Tuple

import numpy as np

from ..utils.data_utils import DataUtilities


class MultiModalDataLoadingMixin:
    """Expects ``self.config`` (a ``DatasetConfig``)."""

    def _resolve(self, path: str, data_folder: Optional[str]) -> str:
        if data_folder and not os.path.isabs(path) and "://" not in path:
            return os.path.join(data_folder, path)
        return path

    # ---- object storage ------------------------------------------------------------------------
    def storage(self):
        """Client for ``config.object_storage`` / ``config.bucket_name`` (``None`` for local files), built on first
        use in the process that reads the data (dataloader workers each get their own)."""
        kind = getattr(self.config, "object_storage", "none")
        if kind in (None, "none", ""):
            return None
        cached = self.__dict__.get("_storage_client")
        if cached is None or cached[0] != os.getpid():
            from ..utils.object_storage import make_client

            cached = (os.getpid(), make_client(kind, getattr(self.config, "bucket_name", None)))
            self.__dict__["_storage_client"] = cached
        return cached[1]

    def open_object(self, blob: str) -> io.BytesIO:
        """In-memory stream of a blob of the configured bucket."""
        from ..utils.object_storage import fetch_stream

        client = self.storage()
        if client is None:
            raise ValueError("open_object needs dataset_config.object_storage (gcs | azure | a registered back end)")
        return fetch_stream(client, blob)

    def local_copy(self, full: str) -> str:
        """A path that decoders can open: the file itself, or a cached download of the blob."""
        client = self.storage()
        if client is None:
            return full
        from ..utils.object_storage import fetch_to_cache

        return fetch_to_cache(client, full, (getattr(self.config, "extra_kwargs", None) or {}).get("object_cache_dir"))

    def load_image(self, path: str, data_folder: Optional[str] = None):
        from PIL import Image

        full = self._resolve(path, data_folder)
        if self.storage() is not None:
            return Image.open(self.open_object(full)).convert("RGB")
        return Image.open(full).convert("RGB")

    def load_audio(self, path: str, sr: int = 16000, data_folder: Optional[str] = None) -> Tuple[np.ndarray, int]:
        full = self._resolve(path, data_folder)
        if self.storage() is not None:
            full = self.local_copy(full)
        try:
            import soundfile as sf

            wav, rate = sf.read(full, dtype="float32", always_2d=False)
        except ImportError:
            with wave.open(full, "rb") as w:
                rate = w.getframerate()
                raw = w.readframes(w.getnframes())
                width = w.getsampwidth()
                wav = np.frombuffer(raw, dtype={1: np.uint8, 2: np.int16, 4: np.int32}[width]).astype(np.float32)
                wav = wav / float(2 ** (8 * width - 1))
                if w.getnchannels() > 1:
                    wav = wav.reshape(-1, w.getnchannels()).mean(-1)
        if wav.ndim > 1:
            wav = wav.mean(-1)
        if rate != sr:
            n = int(round(len(wav) * sr / rate))
            wav = np.interp(np.linspace(0, len(wav) - 1, n), np.arange(len(wav)), wav).astype(np.float32)
        return wav, sr

    def sample_indices(self, total: int, video_fps: float) -> np.ndarray:
        cfg = self.config
        if getattr(cfg, "video_sampling_strategy", "fps") == "frame_num":
            n = DataUtilities.smart_nframes(total, video_fps, nframes=cfg.frame_num, max_frames=cfg.video_max_frames or 768)
        else:
            n = DataUtilities.smart_nframes(total, video_fps, fps=cfg.fps, max_frames=cfg.video_max_frames or 768)
        return np.linspace(0, max(total - 1, 0), n).round().astype(np.int64)

    def load_video(self, path: str, data_folder: Optional[str] = None, video_start: Optional[float] = None,
                   video_end: Optional[float] = None) -> Tuple[np.ndarray, float]:
        """Frames ``[n, H, W, 3] uint8`` and the sampled frames-per-second."""
        full = self.local_copy(self._resolve(path, data_folder))
        backend = getattr(self.config, "video_backend", "qwen_vl_utils")
        if backend == "decord":
            try:
                return self._load_decord(full, video_start, video_end)
            except ImportError:
                pass
        if backend in ("qwen_vl_utils", "qwen_omni_utils"):
            try:
                return self._load_qwen_utils(full, backend, video_start, video_end)
            except ImportError:
                pass
        return self._load_cv2(full, video_start, video_end)

    def load_video_with_metadata(self, path: str, data_folder: Optional[str] = None, video_start: Optional[float] = None,
                                 video_end: Optional[float] = None) -> Tuple[np.ndarray, dict]:
        """Frames plus what a processor needs to talk about time: ``video_time`` (seconds of the source), ``fps`` of
        the source, ``frames_indices`` and ``frame_times`` of the sampled frames, ``total_num_frames`` and the
        effective ``sample_fps``.  Decoded with decord when it is installed, with OpenCV otherwise."""
        full = self.local_copy(self._resolve(path, data_folder))
        try:
            import decord

            vr = decord.VideoReader(full)
            fps, total = float(vr.get_avg_fps()), len(vr)
            read = lambda idx: vr.get_batch(idx).asnumpy()  # noqa: E731
        except ImportError:
            import cv2

            cap = cv2.VideoCapture(full)
            if not cap.isOpened():
                raise FileNotFoundError(full)
            fps = float(cap.get(cv2.CAP_PROP_FPS) or 25.0)
            total = int(cap.get(cv2.CAP_PROP_FRAME_COUNT))

            def read(idx):
                out = []
                for i in idx:
                    cap.set(cv2.CAP_PROP_POS_FRAMES, i)
                    ok, fr = cap.read()
                    if not ok:
                        break
                    out.append(cv2.cvtColor(fr, cv2.COLOR_BGR2RGB))
                cap.release()
                if not out:
                    raise RuntimeError(f"no frames decoded from {full}")
                return np.stack(out)
        lo = int((video_start or 0) * fps)
        hi = min(total, int(video_end * fps)) if video_end else total
        idx = (self.sample_indices(max(hi - lo, 1), fps) + lo).tolist()
        frames = read(idx)
        idx = idx[: len(frames)]
        span = max((hi - lo) / fps, 1e-6)
        return frames, {"video_time": total / fps, "fps": fps, "frames_indices": idx, "frame_times": [i / fps for i in idx],
                        "total_num_frames": total, "sample_fps": len(idx) / span}

    def _load_decord(self, full, start, end):
        import decord

        vr = decord.VideoReader(full)
        fps = float(vr.get_avg_fps())
        lo = int((start or 0) * fps)
        hi = int(end * fps) if end else len(vr)
        idx = self.sample_indices(hi - lo, fps) + lo
        frames = vr.get_batch(idx.tolist()).asnumpy()
        return frames, len(idx) / max((hi - lo) / fps, 1e-6)

    def _load_qwen_utils(self, full, backend, start, end):
        mod = __import__(backend)
        ele = {"type": "video", "video": full, "fps": self.config.fps, "max_frames": self.config.video_max_frames}
        if start is not None:
            ele["video_start"] = start
        if end is not None:
            ele["video_end"] = end
        video, fps = mod.fetch_video(ele, return_video_sample_fps=True)
        arr = video.permute(0, 2, 3, 1).numpy().astype(np.uint8) if hasattr(video, "permute") else np.asarray(video)
        return arr, float(fps)

    def _load_cv2(self, full, start, end):
        import cv2

        cap = cv2.VideoCapture(full)
        if not cap.isOpened():
            raise FileNotFoundError(full)
        fps = cap.get(cv2.CAP_PROP_FPS) or 25.0
        total = int(cap.get(cv2.CAP_PROP_FRAME_COUNT))
        lo = int((start or 0) * fps)
        hi = min(total, int(end * fps)) if end else total
        idx = self.sample_indices(max(hi - lo, 1), fps) + lo
        frames = []
        for i in idx.tolist():
            cap.set(cv2.CAP_PROP_POS_FRAMES, i)
            ok, fr = cap.read()
            if not ok:
                break
            frames.append(cv2.cvtColor(fr, cv2.COLOR_BGR2RGB))
        cap.release()
        if not frames:
            raise RuntimeError(f"no frames decoded from {full}")
        return np.stack(frames), len(frames) / max((hi - lo) / fps, 1e-6)
