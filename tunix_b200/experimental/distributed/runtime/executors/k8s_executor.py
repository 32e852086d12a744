"""Runs process bodies inside pods of an indexed Kubernetes JobSet
(tunix/experimental/distributed/runtime/executors/k8s_executor.py)."""
from __future__ import annotations

from ..contexts import k8s_context
from . import local_executor

K8sProcessContext = k8s_context.K8sProcessContext
pod_dns_name = k8s_context.pod_dns_name


class K8sExecutor(local_executor.LocalExecutor):
  context_cls = k8s_context.K8sProcessContext
