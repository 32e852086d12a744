"""Native rollout engine: paged KV cache, continuous batching, CUDA-graph decode."""
from .engine import EngineConfig, GenerationResult, PagedEngine  # noqa: F401
from .paged_cache import PageAllocator, PagedKVCache, PagedLayerCache  # noqa: F401
