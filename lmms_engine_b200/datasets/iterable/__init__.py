from .multimodal_iterable_dataset import MultiModalIterableDataset  # noqa: F401
