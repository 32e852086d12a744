"""Trajectory schema and stores."""
from .trajectory import *  # noqa: F401,F403
from .store import (TrajectoryMetadataNotFoundError, TrajectoryNotFoundError,
                    TrajectoryReader, TrajectoryWriter)
from .in_memory_store import InMemoryTrajectoryStore
from .file_store import FileTrajectoryStore
from .async_writer import AsyncFileWriter
