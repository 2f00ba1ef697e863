"""The peer-memory all-reduce on ONE GPU, with a CPU thread playing the second rank.

Every buffer and flag pad lives in pinned (device-mapped) host memory, so the CPU peer can speak the kernel's protocol
directly: raise its entry flag, reduce its half of the rows, raise its exit flag.  The second test leaves the peer silent:
the kernel's bounded wait must run out, record the flag-timeout status and return, with the context still usable.
"""
import ctypes
import threading
import time

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
VP = ctypes.c_void_p
WORLD = 2
SLOTS = 8            # flag slots per block row in a pad (one per possible rank)


def _setup(timeout_ms):
    from blaze_b200.ops import get_ops
    ops = get_ops("cuda")
    lib = ops.lib
    lib.blz_comm_create.restype = VP
    lib.blz_comm_create.argtypes = [ctypes.c_int, ctypes.c_int, VP, VP, ctypes.c_int]
    lib.blz_comm_allreduce.argtypes = [VP, VP, VP, VP, VP, ctypes.c_longlong, ctypes.c_int, VP]
    lib.blz_comm_destroy.argtypes = [VP]
    pad_words = int(lib.blz_comm_pad_bytes()) // 4
    pads = [torch.zeros(pad_words, dtype=torch.int32, pin_memory=True) for _ in range(WORLD)]
    epoch = torch.zeros(int(lib.blz_comm_epoch_bytes()) // 4, dtype=torch.int32, device="cuda")
    arr = (VP * WORLD)(*[VP(p.data_ptr()) for p in pads])
    comm = lib.blz_comm_create(0, WORLD, arr, VP(epoch.data_ptr()), timeout_ms)
    assert comm
    return ops, lib, comm, pads, epoch


def test_allreduce_with_a_cpu_thread_as_the_peer():
    ops, lib, comm, pads, epoch = _setup(timeout_ms=5000)
    blocks, n = 4, 64 * 1024                      # bf16 elements; two ranks -> each reduces half
    g = torch.Generator().manual_seed(9)
    ins = [(torch.randn(n, generator=g) * 0.5).bfloat16().pin_memory() for _ in range(WORLD)]
    outs = [torch.zeros(n, dtype=torch.bfloat16).pin_memory() for _ in range(WORLD)]
    want = (ins[0].float() + ins[1].float()).bfloat16()
    failed = []

    def peer():
        """Rank 1 on the CPU: flags go into rank 0's pad at slot 1; rank 0's flags arrive in pads[1] at slot 0."""
        mine, theirs = pads[1].numpy(), pads[0].numpy()
        deadline = time.monotonic() + 20
        for b in range(blocks):                   # entry: the partial sums are ready
            theirs[b * SLOTS + 1] = 1
        while any(mine[b * SLOTS + 0] < 1 for b in range(blocks)):
            if time.monotonic() > deadline:
                failed.append("rank 0 never entered")
                return
            time.sleep(0.0005)
        half = n // 2                              # rank 1 owns the second half of the 16-byte vectors
        s = (ins[0][half:].float() + ins[1][half:].float()).bfloat16()
        outs[0][half:] = s
        outs[1][half:] = s
        for b in range(blocks):                   # exit: my slice is written everywhere
            theirs[b * SLOTS + 1] = 2

    th = threading.Thread(target=peer)
    th.start()
    in_ptrs = (VP * WORLD)(*[VP(t.data_ptr()) for t in ins])
    out_ptrs = (VP * WORLD)(*[VP(t.data_ptr()) for t in outs])
    rc = lib.blz_comm_allreduce(comm, in_ptrs, out_ptrs, VP(0), VP(0), n * 2, blocks,
                                VP(torch.cuda.current_stream().cuda_stream))
    assert rc == 0
    torch.cuda.synchronize()
    th.join(timeout=30)
    assert not failed and not th.is_alive()
    assert ops.take_status() == 0
    assert torch.equal(outs[0], want) and torch.equal(outs[1], want)
    lib.blz_comm_destroy(comm)


def test_silent_peer_runs_the_wait_out_and_reports_it():
    ops, lib, comm, pads, epoch = _setup(timeout_ms=300)
    n = 4096
    ins = [torch.ones(n, dtype=torch.bfloat16).pin_memory() for _ in range(WORLD)]
    outs = [torch.zeros(n, dtype=torch.bfloat16).pin_memory() for _ in range(WORLD)]
    in_ptrs = (VP * WORLD)(*[VP(t.data_ptr()) for t in ins])
    out_ptrs = (VP * WORLD)(*[VP(t.data_ptr()) for t in outs])
    t0 = time.monotonic()
    rc = lib.blz_comm_allreduce(comm, in_ptrs, out_ptrs, VP(0), VP(0), n * 2, 2, VP(torch.cuda.current_stream().cuda_stream))
    assert rc == 0
    torch.cuda.synchronize()                      # returns: the wait is bounded
    assert time.monotonic() - t0 < 10
    assert ops.take_status() == 2                 # flag wait ran out
    assert int(outs[0].float().abs().sum()) == 0  # nothing was reduced after the failed entry barrier
    # the context is still usable, and the next kernel of this communicator is in step with its epochs
    x = torch.ones(8, device="cuda") * 2
    assert float(x.sum()) == 16.0
    assert ops.take_status() == 0
    lib.blz_comm_destroy(comm)
