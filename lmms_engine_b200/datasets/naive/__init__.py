from .multimodal_dataset import MultiModalDataset  # noqa: F401
