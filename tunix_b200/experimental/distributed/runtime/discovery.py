"""TCP peer discovery used by the local and Kubernetes process contexts.

A process started with a discovery port listens there; peers started with that
address connect, send one length-prefixed frame (their own id, port and opaque
metadata) and wait for a one-byte acknowledgement. Registration retries until a
deadline, so start order does not matter. Frames are plain bytes: nothing is
unpickled from the network.
"""

from __future__ import annotations

import logging
import socket
import struct
import threading
import time
from typing import Callable

from . import context

log = logging.getLogger(__name__)
_MAX_FRAME = 16 << 20


def _recv_exact(conn: socket.socket, n: int) -> bytes:
  buf = bytearray()
  while len(buf) < n:
    chunk = conn.recv(n - len(buf))
    if not chunk:
      raise ConnectionError("peer closed during a frame")
    buf += chunk
  return bytes(buf)


def encode_frame(host: str, port: int, metadata: bytes) -> bytes:
  h = host.encode("utf-8")
  body = struct.pack("!HI", len(h), port) + h + metadata
  return struct.pack("!I", len(body)) + body


def decode_frame(body: bytes) -> tuple[str, int, bytes]:
  hlen, port = struct.unpack("!HI", body[:6])
  return body[6:6 + hlen].decode("utf-8"), port, body[6 + hlen:]


def parse_addrs(addrs: str) -> list[tuple[str, int]]:
  out = []
  for item in filter(None, (a.strip() for a in addrs.split(","))):
    host, _, port = item.rpartition(":")
    if not host or not port.isdigit():
      raise ValueError(f"discovery address '{item}' is not host:port")
    out.append((host, int(port)))
  return out


class TcpDiscovery(context.DiscoveryContext):

  def __init__(self, my_id: str, my_port: int, peer_addrs: str = "",
               bind_host: str = "0.0.0.0",
               resolve: Callable[[str], str] | None = None,
               register_timeout: float = 60.0):
    self._id = my_id or socket.gethostname()
    self._port = int(my_port)
    self._peers = parse_addrs(peer_addrs)
    self._bind_host = bind_host
    self._resolve = resolve or (lambda h: h)
    self._timeout = register_timeout
    self._callbacks: list[Callable[[str, int, bytes], None]] = []
    self._seen: list[tuple[str, int, bytes]] = []
    self._lock = threading.Lock()
    self._server: socket.socket | None = None
    self._thread: threading.Thread | None = None
    self._stop = threading.Event()

  # -- server ---------------------------------------------------------------

  def start(self) -> None:
    if not self._port or self._server is not None:
      return
    srv = socket.socket(socket.AF_INET, socket.SOCK_STREAM)
    srv.setsockopt(socket.SOL_SOCKET, socket.SO_REUSEADDR, 1)
    srv.bind((self._bind_host, self._port))
    srv.listen(128)
    srv.settimeout(0.2)
    self._server = srv
    self._port = srv.getsockname()[1]
    self._thread = threading.Thread(target=self._serve, daemon=True,
                                    name=f"discovery-{self._id}")
    self._thread.start()

  @property
  def port(self) -> int:
    return self._port

  def is_started(self) -> bool:
    return self._server is not None and not self._stop.is_set()

  def _serve(self) -> None:
    while not self._stop.is_set():
      try:
        conn, _ = self._server.accept()
      except socket.timeout:
        continue
      except OSError:
        return
      with conn:
        try:
          conn.settimeout(5.0)
          (n,) = struct.unpack("!I", _recv_exact(conn, 4))
          if n > _MAX_FRAME:
            raise ValueError(f"frame of {n} bytes refused")
          peer = decode_frame(_recv_exact(conn, n))
          conn.sendall(b"\x01")
        except Exception:  # pylint: disable=broad-exception-caught
          log.exception("discovery: bad registration dropped")
          continue
      with self._lock:
        self._seen.append(peer)
        callbacks = list(self._callbacks)
      for cb in callbacks:
        try:
          cb(*peer)
        except Exception:  # pylint: disable=broad-exception-caught
          log.exception("discovery: on_register callback raised")

  def stop(self) -> None:
    self._stop.set()
    if self._server is not None:
      try:
        self._server.close()
      except OSError:
        pass
    if self._thread is not None:
      self._thread.join(2.0)

  # -- DiscoveryContext -------------------------------------------------------

  def on_register(self, callback) -> None:
    with self._lock:
      self._callbacks.append(callback)
      replay = list(self._seen)
    for peer in replay:
      callback(*peer)

  def register(self, metadata: bytes) -> None:
    frame = encode_frame(self._id, self._port, metadata)
    for host, port in self._peers:
      deadline = time.monotonic() + self._timeout
      delay = 0.05
      while True:
        try:
          with socket.create_connection((self._resolve(host), port),
                                        timeout=2.0) as c:
            c.sendall(frame)
            if _recv_exact(c, 1) != b"\x01":
              raise ConnectionError("registration not acknowledged")
          break
        except OSError as e:
          if time.monotonic() >= deadline:
            raise TimeoutError(
                f"could not register with {host}:{port} within"
                f" {self._timeout:.0f}s: {e}") from e
          time.sleep(delay)
          delay = min(delay * 2, 1.0)
