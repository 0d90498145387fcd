"""Token-stream datasets and loaders."""

from nestor_b200.data.datasets import DclmTokenDataset, PinnedWindowLoader, build_dataset, write_synthetic_bin  # noqa: F401
