"""Runs process bodies inside pods of an indexed Kubernetes JobSet.

A discovery id names a replicated job; its address is the stable DNS name the
JobSet controller gives pod 0 of that job:
``<jobset>-<job>-0-0.<jobset>``. Rank and world size come from the JobSet's
completion index and the ``TUNIX_*`` variables the deployment templates set.
"""

from __future__ import annotations

import os

from . import local_executor


def pod_dns_name(jobset: str, job: str, job_index: int = 0,
                 pod_index: int = 0) -> str:
  return f"{jobset}-{job}-{job_index}-{pod_index}.{jobset}"


class K8sProcessContext(local_executor.LocalProcessContext):

  def __init__(self, context_args, environ=None):
    self._env = os.environ if environ is None else environ
    self._jobset = self._env.get("JOBSET_NAME", "")
    if "RANK" not in self._env and "JOB_COMPLETION_INDEX" in self._env:
      nodes = int(self._env.get("TUNIX_NUM_NODES", "1"))
      per = int(self._env.get("TUNIX_GPUS_PER_NODE", "1"))
      local = int(self._env.get("LOCAL_RANK", "0"))
      os.environ["RANK"] = str(
          int(self._env["JOB_COMPLETION_INDEX"]) * per + local)
      os.environ["WORLD_SIZE"] = str(nodes * per)
    if "MASTER_ADDR" not in self._env and self._jobset:
      os.environ["MASTER_ADDR"] = pod_dns_name(
          self._jobset, self._env.get("REPLICATED_JOB_NAME", "proc"))
    super().__init__(context_args)

  def _bind_host(self) -> str:
    return "0.0.0.0"

  def _resolve(self, host: str) -> str:
    if "." in host or not self._jobset:
      return host
    return pod_dns_name(self._jobset, host)


class K8sExecutor(local_executor.LocalExecutor):
  context_cls = K8sProcessContext
