"""Process executors (tunix/experimental/distributed/runtime/executor.py)."""
from .executors.k8s_executor import K8sExecutor
from .executors.local_executor import LocalExecutor
