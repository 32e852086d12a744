"""A device-side wait that nothing satisfies ends by itself and reports through the status word."""

import time

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_peer_barrier_gives_up_and_context_survives():
  from tunix_b200.ops import _lib
  from tunix_b200.dist import symm
  lib = symm._declare()     # pointer-typed signatures: an undeclared ctypes call would truncate addresses
  dev = torch.device("cuda", 0)
  # Two flag rows on one GPU stand in for two ranks; "rank 1" never arrives.
  rows = [torch.zeros(16, dtype=torch.int32, device=dev) for _ in range(2)]
  status = _lib.status_word(dev)
  status.zero_()
  torch.cuda.synchronize()
  t0 = time.time()
  rc = lib.tx_peer_barrier(symm._ptr_array([r.data_ptr() for r in rows]), 0, 2, 1, 300,
                           status.data_ptr(), _lib.stream_ptr())
  assert rc == 0
  torch.cuda.synchronize()
  waited = time.time() - t0
  assert 0.25 < waited < 5.0
  assert int(rows[1][0]) == 1          # our arrival was published to the peer's row
  with pytest.raises(RuntimeError, match="0x10"):
    _lib.check_status(dev)
  _lib.check_status(dev)               # the word was cleared
  # the context is still usable, and a barrier whose peer did arrive passes
  rows[0][1] = 2
  rc = lib.tx_peer_barrier(symm._ptr_array([r.data_ptr() for r in rows]), 0, 2, 2, 300,
                           status.data_ptr(), _lib.stream_ptr())
  assert rc == 0
  torch.cuda.synchronize()
  _lib.check_status(dev)
  assert float((torch.ones(8, device=dev) * 2).sum()) == 16.0


def test_device_lane_span_is_closed_by_a_cuda_timing_event(kernel_lib):
  """A device-lane span over CUDA work ends at the device timestamp of an event recorded behind the work, mapped
  onto the host clock; no waiter thread is involved."""
  import time
  from tunix_b200.perf.experimental import timeline
  lane = timeline.AsyncTimeline("cuda0", time.perf_counter())
  a = torch.randn(4096, 4096, device="cuda")
  torch.cuda.synchronize()
  e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
  begin = time.perf_counter()
  e0.record()
  for _ in range(20):
    a = a @ a * 1e-3
  e1.record()
  lane.span("work", begin, [a])
  assert lane._resolver is None and not lane.cur_step          # nothing resolved, nothing blocked yet
  lane.wait_pending_spans()
  (span,) = lane.cur_step.values()
  device_s = e0.elapsed_time(e1) * 1e-3
  assert span.ended and span.duration >= 0.8 * device_s and span.duration < device_s + 0.05


def test_own_peer_allocator_single_rank(kernel_lib, tmp_path):
  """`dist/vmm.py` with a group of one: the buffer is a real tensor over driver-allocated memory, and the 2-D peer
  copy kernel reads it through the pointer the heap reports."""
  import torch.distributed as dist
  from tunix_b200.dist import symm, vmm
  assert vmm.available() is None
  created = not dist.is_initialized()
  if created:
    dist.init_process_group("gloo", init_method=f"file://{tmp_path}/rdv", rank=0, world_size=1)
  try:
    dev = torch.device("cuda", 0)
    heap = vmm.PeerHeap(None, dev)
    buf = heap.alloc(4096 * 2)
    t = buf.local.view(torch.bfloat16)
    assert t.numel() == 4096 and t.data_ptr() == buf.ptrs[0] and float(t.float().abs().sum()) == 0.0
    t.copy_(torch.arange(4096, device=dev).to(torch.bfloat16))
    lib = symm._declare()
    from tunix_b200.ops import _lib
    dst = torch.zeros(8, 256, dtype=torch.bfloat16, device=dev)
    rc = lib.tx_peer_copy_2d(buf.ptrs[0] + 2 * 256, dst.data_ptr(), 8, 256, 512, 256, _lib.stream_ptr())
    assert rc == 0
    torch.cuda.synchronize()
    assert torch.equal(dst, t.view(8, 512)[:, 256:])
    heap.close()
  finally:
    if created:
      dist.destroy_process_group()
