"""In-memory datasets with the map/filter/slice/repeat/batch surface the CLI and examples use."""
from .dataset import IterDataset, ListDataset, default_batch_fn  # noqa: F401
