"""Object-storage access for the data plane: media named by ``bucket`` + blob path are fetched into
memory (images, audio) or into a per-process cache file (videos, which the decoders open by path).

``dataset_config.object_storage``: ``gcs`` (google-cloud-storage), ``azure`` (azure-storage-blob; account URL /
SAS from ``AZURE_STORAGE_SAS_URL``) or ``none``.  The SDKs are imported only when a dataset asks for them.
``register_storage_backend`` adds further back ends (and lets tests stand one up without a network).
Downloads are retried with exponential back-off; a blob that stays unreadable raises, so the dataset's
skip-and-log path handles it like any other damaged record.

Counterpart in the reference: clients built in the dataset constructors and
``DataUtilities.download_blob_to_stream`` (src/lmms_engine/datasets/naive/multimodal_dataset.py:40-55,
src/lmms_engine/utils/data_utils.py:204-227), which logs a failed download and carries on with an
empty stream.
"""
from __future__ import annotations

import hashlib
import io
import os
import tempfile
import time
from typing import Callable, Dict, Optional

from .logging_utils import logger


class StorageClient:
    """Minimal interface: ``read(blob) -> bytes``."""

    def __init__(self, bucket: str):
        self.bucket = bucket

    def read(self, blob: str) -> bytes:  # pragma: no cover - interface
        raise NotImplementedError


class GCSClient(StorageClient):
    def __init__(self, bucket: str):
        super().__init__(bucket)
        try:
            from google.cloud.storage import Client
        except ImportError as e:
            raise ImportError("object_storage: gcs needs the google-cloud-storage package") from e
        self._bucket = Client().bucket(bucket)

    def read(self, blob: str) -> bytes:
        return self._bucket.blob(blob).download_as_bytes()


class AzureClient(StorageClient):
    def __init__(self, bucket: str):
        super().__init__(bucket)
        try:
            from azure.storage.blob import BlobServiceClient
        except ImportError as e:
            raise ImportError("object_storage: azure needs the azure-storage-blob package") from e
        url = os.environ.get("AZURE_STORAGE_SAS_URL")
        if not url:
            raise ValueError("object_storage: azure needs AZURE_STORAGE_SAS_URL (account URL with a SAS token)")
        self._svc = BlobServiceClient(account_url=url)

    def read(self, blob: str) -> bytes:
        return self._svc.get_blob_client(container=self.bucket, blob=blob).download_blob().readall()


class LocalDirectoryClient(StorageClient):
    """``bucket`` is a directory: the same code path as a remote store, for tests and air-gapped mirrors."""

    def read(self, blob: str) -> bytes:
        with open(os.path.join(self.bucket, blob), "rb") as f:
            return f.read()


_BACKENDS: Dict[str, Callable[[str], StorageClient]] = {"gcs": GCSClient, "azure": AzureClient, "local": LocalDirectoryClient}


def register_storage_backend(name: str, factory: Callable[[str], StorageClient]) -> None:
    _BACKENDS[name] = factory


def make_client(kind: Optional[str], bucket: Optional[str]) -> Optional[StorageClient]:
    if kind in (None, "none", ""):
        return None
    if kind not in _BACKENDS:
        raise ValueError(f"unknown object_storage '{kind}'; known: {sorted(_BACKENDS)}")
    if not bucket:
        raise ValueError(f"object_storage: {kind} needs dataset_config.bucket_name")
    return _BACKENDS[kind](bucket)


def fetch(client: StorageClient, blob: str, retries: int = 5, backoff: float = 0.5) -> bytes:
    last: Optional[Exception] = None
    for attempt in range(max(retries, 1)):
        try:
            return client.read(blob)
        except Exception as e:  # noqa: BLE001 - SDK errors are not one hierarchy
            last = e
            logger.warning(f"object storage: attempt {attempt + 1}/{retries} for {client.bucket}/{blob} failed: {type(e).__name__}: {e}")
            if attempt + 1 < retries:
                time.sleep(backoff * (2 ** attempt))
    raise IOError(f"object storage: could not read {client.bucket}/{blob}") from last


def fetch_stream(client: StorageClient, blob: str, **kw) -> io.BytesIO:
    return io.BytesIO(fetch(client, blob, **kw))


def fetch_to_cache(client: StorageClient, blob: str, cache_dir: Optional[str] = None, **kw) -> str:
    """Local path of the blob (downloaded once per process tree into ``cache_dir``): video decoders want files."""
    root = cache_dir or os.path.join(tempfile.gettempdir(), "lmms_engine_b200_objects")
    os.makedirs(root, exist_ok=True)
    name = hashlib.sha1(f"{client.bucket}/{blob}".encode()).hexdigest() + os.path.splitext(blob)[1]
    path = os.path.join(root, name)
    if not os.path.exists(path):
        data = fetch(client, blob, **kw)
        tmp = f"{path}.{os.getpid()}.part"
        with open(tmp, "wb") as f:
            f.write(data)
        os.replace(tmp, path)
    return path
