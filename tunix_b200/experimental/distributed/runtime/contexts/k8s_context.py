"""Process context for pods of an indexed Kubernetes JobSet
(tunix/experimental/distributed/runtime/contexts/k8s_context.py:27-216).

Names come from the JobSet controller's stable DNS scheme `<jobset>-<job>-<job index>-<pod index>.<jobset>`:

  * a discovery id names a replicated job, and its address is pod 0 of job 0 of it;
  * a pod announces itself to peers under its own such name, built from the JOBSET_NAME / REPLICATED_JOB_NAME /
    JOB_INDEX / POD_INDEX variables of the pod template;
  * rank and world size, when the launcher did not set them, follow from the pod's completion index and the
    TUNIX_NUM_NODES / TUNIX_GPUS_PER_NODE variables; the rendezvous address defaults to pod 0 of this pod's job.
"""
from __future__ import annotations

import os
from typing import Any, Mapping, Optional

from . import local_context

_POD_VARIABLES = ("JOBSET_NAME", "REPLICATED_JOB_NAME", "JOB_INDEX", "POD_INDEX")


def pod_dns_name(jobset: str, job: str, job_index: int = 0, pod_index: int = 0) -> str:
  return f"{jobset}-{job}-{job_index}-{pod_index}.{jobset}"


def resolve_discovery_address(discovery_address: str, jobset: Optional[str] = None) -> str:
  """'door:12345' -> '<pod 0 of job door>:12345'. Without `jobset` the id is its own jobset with the single
  replicated job `proc` (the layout the deployment templates produce for a one-job set)."""
  discovery_id, _, port = discovery_address.rpartition(":")
  if not discovery_id or not port.isdigit():
    raise ValueError(f"discovery address '{discovery_address}' is not id:port")
  host = pod_dns_name(jobset, discovery_id) if jobset else pod_dns_name(discovery_id, "proc")
  return f"{host}:{port}"


def resolve_self_hostname(environ: Optional[Mapping[str, str]] = None) -> str:
  env = os.environ if environ is None else environ
  missing = [v for v in _POD_VARIABLES if v not in env]
  if missing:
    raise ValueError(f"Missing required environment variable(s): {', '.join(missing)}")
  return pod_dns_name(env["JOBSET_NAME"], env["REPLICATED_JOB_NAME"], env["JOB_INDEX"], env["POD_INDEX"])


class K8sIpcContext(local_context.LocalIpcContext):
  pass


class K8sProcessContext(local_context.LocalProcessContext):

  ipc_cls = K8sIpcContext

  def __init__(self, context_args: Any, environ: Optional[Mapping[str, str]] = None):
    self._env = os.environ if environ is None else environ
    self._jobset = self._env.get("JOBSET_NAME", "")
    if "RANK" not in self._env and "JOB_COMPLETION_INDEX" in self._env:
      nodes = int(self._env.get("TUNIX_NUM_NODES", "1"))
      per = int(self._env.get("TUNIX_GPUS_PER_NODE", "1"))
      local = int(self._env.get("LOCAL_RANK", "0"))
      os.environ["RANK"] = str(int(self._env["JOB_COMPLETION_INDEX"]) * per + local)
      os.environ["WORLD_SIZE"] = str(nodes * per)
    if "MASTER_ADDR" not in self._env and self._jobset:
      os.environ["MASTER_ADDR"] = pod_dns_name(self._jobset, self._env.get("REPLICATED_JOB_NAME", "proc"))
    super().__init__(context_args)

  def _own_name(self, discovery_id: str) -> str:
    try:
      return resolve_self_hostname(self._env)        # peers can connect back to this
    except ValueError:
      return discovery_id

  def _bind_host(self) -> str:
    return "0.0.0.0"

  def _resolve(self, host: str) -> str:
    if "." in host or not self._jobset:
      return host
    return pod_dns_name(self._jobset, host)
