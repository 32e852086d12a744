"""Weight-sync transport between OS jobs that share no process group: device -> pinned host -> TCP -> pinned host ->
device. This is the role the reference's internal host-staged transport plays
(tunix/experimental/orchestrator/raiden_handler.py:49-550, tunix/experimental/worker/raiden_synchronizer.py:30-277);
inside one job the peer-memory kernel (`dist/weight_sync.py`) or `PeerMemoryHandler` are the faster paths.

Two parts, split the way the protocol splits control from data:

`HostStagedEndpoint` runs in every process that holds weights - the trainer (its prepared tensors) and each rollout
worker (its STAGING tensors). It is a small TCP server on its own thread and answers

  fetch     streams the named tensors of an attached unit: per tensor a JSON header, then the raw bytes. CUDA tensors
            go through two pinned host buffers, so the device-to-host copy of tensor k+1 overlaps the send of k;
  pull      "fill your unit X from unit Y at address A": the endpoint connects to A, fetches exactly the tensors its
            own unit has, receives into pinned buffers and copies host-to-device asynchronously, again two deep;
  checksum  SHA-256 over a unit's bytes (verification after a round, tests);
  describe / ping.

`HostStagedHandler` is the `WeightSyncHandler` the coordinator holds. It owns no tensors: `transfer` checks the
registered manifests against each other, then tells every destination endpoint to pull from the source endpoint, all
destinations in parallel, and folds their answers into one `TransferResult`. A destination that cannot be reached
before anything was sent is a known failure; a connection that dies or times out after the command went out leaves
the staging copy in an unknown state and raises `TransferOutcomeUnknownError`, which the coordinator treats as such.

A fetch names the generation it expects; an endpoint whose unit was attached for another generation refuses, so a
late round cannot read half-replaced weights. Every socket operation has a deadline.
"""
from __future__ import annotations

import concurrent.futures
import contextlib
import hashlib
import json
import socket
import struct
import threading
from typing import Any, Dict, List, Mapping, Optional, Sequence, Tuple, Union

import torch

from . import weight_sync

Address = Tuple[str, int]
_HEADER = struct.Struct(">I")


def unit_key(unit: Union[weight_sync.WorkUnitId, str]) -> str:
  if isinstance(unit, str):
    return unit
  return f"{unit.job_name}/{unit.job_replica_id}/{unit.data_replica_idx}"


# ---- framing ---------------------------------------------------------------------------------------
def _send_json(sock: socket.socket, obj: Mapping[str, Any]) -> None:
  body = json.dumps(obj).encode("utf-8")
  sock.sendall(_HEADER.pack(len(body)) + body)


def _recv_exact(sock: socket.socket, view: memoryview) -> None:
  got = 0
  while got < len(view):
    n = sock.recv_into(view[got:])
    if n == 0:
      raise ConnectionError(f"peer closed the connection after {got} of {len(view)} bytes")
    got += n


def _recv_json(sock: socket.socket) -> Dict[str, Any]:
  head = bytearray(_HEADER.size)
  _recv_exact(sock, memoryview(head))
  body = bytearray(_HEADER.unpack(head)[0])
  _recv_exact(sock, memoryview(body))
  return json.loads(body.decode("utf-8"))


def _bytes_of(t: torch.Tensor) -> torch.Tensor:
  """Flat uint8 view of a contiguous tensor's storage (works for bf16, which NumPy cannot name)."""
  return t.detach().contiguous().view(-1).view(torch.uint8) if t.numel() else torch.empty(0, dtype=torch.uint8)


class _PinnedPair:
  """Two host buffers that grow on demand; pinned when a GPU is present."""

  def __init__(self):
    self._bufs: List[Optional[torch.Tensor]] = [None, None]
    self._pin = torch.cuda.is_available()

  def get(self, slot: int, nbytes: int) -> torch.Tensor:
    buf = self._bufs[slot]
    if buf is None or buf.numel() < nbytes:
      buf = torch.empty(max(nbytes, 1), dtype=torch.uint8, pin_memory=self._pin)
      self._bufs[slot] = buf
    return buf[:nbytes]


class HostStagedEndpoint:

  def __init__(self, host: str = "127.0.0.1", port: int = 0, timeout_s: float = 60.0):
    self._timeout = float(timeout_s)
    self._units: Dict[str, Tuple[Mapping[str, torch.Tensor], Optional[int]]] = {}
    self._lock = threading.Lock()
    self._server = socket.create_server((host, port))
    self._server.settimeout(0.2)
    self.address: Address = self._server.getsockname()[:2]
    self._closing = threading.Event()
    self._thread = threading.Thread(target=self._accept_loop, daemon=True, name="host-staged-endpoint")
    self._thread.start()
    self.served = {"fetch": 0, "pull": 0}

  # ---- what this process offers ------------------------------------------------------------------
  def attach(self, unit: Union[weight_sync.WorkUnitId, str], tensors: Mapping[str, torch.Tensor],
             generation: Optional[int] = None) -> None:
    """Sources attach the prepared weights of a round, destinations their staging copy. `generation` (when given)
    is what a fetch must name to be served."""
    with self._lock:
      self._units[unit_key(unit)] = (tensors, generation)

  def detach(self, unit: Union[weight_sync.WorkUnitId, str]) -> None:
    with self._lock:
      self._units.pop(unit_key(unit), None)

  def close(self) -> None:
    self._closing.set()
    self._thread.join(timeout=2.0)
    self._server.close()

  def __enter__(self) -> "HostStagedEndpoint":
    return self

  def __exit__(self, *exc) -> None:
    self.close()

  # ---- server ------------------------------------------------------------------------------------
  def _accept_loop(self) -> None:
    while not self._closing.is_set():
      try:
        conn, _ = self._server.accept()
      except socket.timeout:
        continue
      except OSError:
        return
      threading.Thread(target=self._serve_one, args=(conn,), daemon=True).start()

  def _serve_one(self, conn: socket.socket) -> None:
    with conn:
      conn.settimeout(self._timeout)
      try:
        request = _recv_json(conn)
        op = request.get("op")
        if op == "ping":
          _send_json(conn, {"ok": True})
        elif op == "describe":
          _send_json(conn, self._describe(request["unit"]))
        elif op == "checksum":
          _send_json(conn, self._checksum(request["unit"]))
        elif op == "fetch":
          self._fetch(conn, request)
        elif op == "pull":
          _send_json(conn, self._pull(request))
        else:
          _send_json(conn, {"ok": False, "message": f"unknown op {op!r}"})
      except Exception as e:  # noqa: BLE001 - reported to the peer when the socket still works
        try:
          _send_json(conn, {"ok": False, "message": f"{type(e).__name__}: {e}"})
        except OSError:
          pass

  def _unit(self, key: str):
    with self._lock:
      if key not in self._units:
        raise KeyError(f"no unit {key!r} is attached to the endpoint at {self.address}")
      return self._units[key]

  def _describe(self, key: str) -> Dict[str, Any]:
    tensors, generation = self._unit(key)
    return {"ok": True, "generation": generation,
            "variables": [{"name": n, "shape": list(t.shape), "dtype": str(t.dtype).replace("torch.", "")}
                          for n, t in tensors.items()]}

  @torch.no_grad()
  def _checksum(self, key: str) -> Dict[str, Any]:
    tensors, _ = self._unit(key)
    digest = hashlib.sha256()
    for name in sorted(tensors):
      digest.update(name.encode("utf-8"))
      digest.update(_bytes_of(tensors[name]).cpu().numpy().tobytes())
    return {"ok": True, "sha256": digest.hexdigest()}

  @torch.no_grad()
  def _fetch(self, conn: socket.socket, request: Mapping[str, Any]) -> None:
    tensors, generation = self._unit(request["unit"])
    wanted = request.get("generation")
    if generation is not None and wanted is not None and int(wanted) != int(generation):
      _send_json(conn, {"ok": False, "message": f"unit {request['unit']!r} is attached for generation {generation}, "
                                                f"the fetch names {wanted}"})
      return
    names = list(request.get("names") or tensors.keys())
    missing = [n for n in names if n not in tensors]
    if missing:
      _send_json(conn, {"ok": False, "message": f"unit {request['unit']!r} has no tensors {missing[:3]}"})
      return
    _send_json(conn, {"ok": True, "count": len(names)})
    pair = _PinnedPair()
    staged: List[Optional[Tuple[torch.Tensor, Optional[torch.cuda.Event]]]] = [None, None]

    def stage(i: int) -> None:
      raw = _bytes_of(tensors[names[i]])
      if not raw.is_cuda:
        staged[i % 2] = (raw, None)
        return
      host = pair.get(i % 2, raw.numel())
      with torch.cuda.device(raw.device):            # this thread's current device is not necessarily the tensor's
        host.copy_(raw, non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
      staged[i % 2] = (host, ev)

    for device in {t.device for t in tensors.values() if t.is_cuda}:
      torch.cuda.synchronize(device)                 # whatever produced the attached tensors has finished
    moved = 0
    if names:
      stage(0)
    for i, name in enumerate(names):
      host, ev = staged[i % 2]
      if i + 1 < len(names):
        stage(i + 1)                      # its copy runs while tensor i is on the wire
      if ev is not None:
        ev.synchronize()
      t = tensors[name]
      _send_json(conn, {"name": name, "dtype": str(t.dtype).replace("torch.", ""), "shape": list(t.shape),
                        "nbytes": host.numel()})
      if host.numel():
        conn.sendall(memoryview(host.numpy()))
      moved += host.numel()
    _send_json(conn, {"done": True, "moved": moved})
    self.served["fetch"] += 1

  @torch.no_grad()
  def _pull(self, request: Mapping[str, Any]) -> Dict[str, Any]:
    staging, _ = self._unit(request["dst_unit"])
    names = list(staging.keys())
    pair = _PinnedPair()
    busy: List[Optional[torch.cuda.Event]] = [None, None]
    moved = 0
    with socket.create_connection(tuple(request["src_addr"]), timeout=self._timeout) as src:
      src.settimeout(self._timeout)
      _send_json(src, {"op": "fetch", "unit": request["src_unit"], "names": names,
                       "generation": request.get("generation")})
      opened = _recv_json(src)
      if not opened.get("ok"):
        return {"ok": False, "moved": 0, "message": opened.get("message", "source refused the fetch")}
      for i in range(int(opened["count"])):
        head = _recv_json(src)
        dst = staging[head["name"]]
        raw = _bytes_of(dst) if dst.is_contiguous() else None
        if tuple(head["shape"]) != tuple(dst.shape):
          return {"ok": False, "moved": moved, "message": f"shape mismatch for {head['name']!r}: source "
                                                          f"{head['shape']} vs staging {list(dst.shape)}"}
        if busy[i % 2] is not None:
          busy[i % 2].synchronize()       # the host buffer's previous upload has finished
          busy[i % 2] = None
        host = pair.get(i % 2, int(head["nbytes"]))
        if host.numel():
          _recv_exact(src, memoryview(host.numpy()))
        with torch.cuda.device(dst.device) if dst.is_cuda else contextlib.nullcontext():
          if raw is not None and head["dtype"] == str(dst.dtype).replace("torch.", ""):
            raw.copy_(host, non_blocking=True)             # same dtype: bytes straight into the staging tensor
          elif host.numel():
            incoming = host.view(getattr(torch, head["dtype"])).view(dst.shape)
            dst.copy_(incoming.to(dst.device, non_blocking=True).to(dst.dtype))
          if dst.is_cuda:
            busy[i % 2] = torch.cuda.Event()
            busy[i % 2].record()
        moved += host.numel()
      tail = _recv_json(src)
      if not tail.get("done"):
        return {"ok": False, "moved": moved, "message": tail.get("message", "source ended the stream early")}
    for ev in busy:
      if ev is not None:
        ev.synchronize()
    self.served["pull"] += 1
    return {"ok": True, "moved": moved, "message": f"{moved} bytes into {request['dst_unit']}"}


def call(address: Address, request: Mapping[str, Any], timeout_s: float = 60.0) -> Dict[str, Any]:
  """One request / one JSON reply to an endpoint."""
  with socket.create_connection(tuple(address), timeout=timeout_s) as sock:
    sock.settimeout(timeout_s)
    _send_json(sock, request)
    return _recv_json(sock)


class HostStagedHandler(weight_sync.WeightSyncHandler):

  def __init__(self, endpoints: Optional[Mapping[Union[weight_sync.WorkUnitId, str], Address]] = None,
               timeout_s: float = 600.0):
    self._timeout = float(timeout_s)
    self._addr: Dict[str, Address] = {unit_key(u): tuple(a) for u, a in (endpoints or {}).items()}
    self._meta: Dict[str, weight_sync.WorkUnitMetadata] = {}
    self._lock = threading.Lock()

  def register_endpoint(self, unit: Union[weight_sync.WorkUnitId, str], address: Address) -> None:
    with self._lock:
      self._addr[unit_key(unit)] = tuple(address)

  def register_work_unit(self, metadata: weight_sync.WorkUnitMetadata) -> None:
    with self._lock:
      self._meta[unit_key(metadata.unit)] = metadata

  def _mismatch(self, src: weight_sync.WorkUnitMetadata, dst: weight_sync.WorkUnitMetadata) -> Optional[str]:
    offered = {v.name: v for v in src.variables}
    for v in dst.variables:
      if v.name not in offered:
        return f"destination {unit_key(dst.unit)} expects {v.name!r}, which the source does not provide"
      if tuple(offered[v.name].shape) != tuple(v.shape):
        return f"shape mismatch for {v.name!r}: source {offered[v.name].shape} vs destination {v.shape}"
    return None

  def transfer(self, src_units, dst_units, req_id=None, generation=None) -> weight_sync.TransferResult:
    rid = req_id or ""
    if not src_units or not dst_units:
      return weight_sync.TransferResult(rid, False, "transfer needs at least one source and one destination unit")
    src = unit_key(src_units[0])
    with self._lock:
      for key in [src] + [unit_key(d) for d in dst_units]:
        if key not in self._meta:
          return weight_sync.TransferResult(rid, False, f"work unit {key} was never registered")
        if key not in self._addr:
          return weight_sync.TransferResult(rid, False, f"work unit {key} has no endpoint address")
      for d in dst_units:
        why = self._mismatch(self._meta[src], self._meta[unit_key(d)])
        if why:
          return weight_sync.TransferResult(rid, False, why)
      src_addr = self._addr[src]
      targets = [(unit_key(d), self._addr[unit_key(d)]) for d in dst_units]

    def command(target) -> Dict[str, Any]:
      key, address = target
      try:
        sock = socket.create_connection(address, timeout=min(self._timeout, 30.0))
      except OSError as e:                                 # nothing was sent: a known failure
        return {"ok": False, "moved": 0, "message": f"destination endpoint {address} unreachable: {e}"}
      with sock:
        sock.settimeout(self._timeout)
        try:
          _send_json(sock, {"op": "pull", "dst_unit": key, "src_unit": src, "src_addr": list(src_addr),
                            "generation": generation, "req_id": rid})
          return _recv_json(sock)
        except (OSError, ConnectionError, ValueError) as e:
          raise weight_sync.TransferOutcomeUnknownError(
              f"pull into {key} at {address}: connection lost after the command was sent ({e})") from e

    with concurrent.futures.ThreadPoolExecutor(max_workers=min(16, len(targets))) as pool:
      answers = list(pool.map(command, targets))
    failed = [f"{key}: {a.get('message', 'failed')}" for (key, _), a in zip(targets, answers) if not a.get("ok")]
    if failed:
      return weight_sync.TransferResult(rid, False, "; ".join(failed))
    moved = sum(int(a.get("moved", 0)) for a in answers)
    return weight_sync.TransferResult(rid, True, f"{moved} bytes to {len(targets)} destination unit(s) over TCP")
