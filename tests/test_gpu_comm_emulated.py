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


def _push_setup(timeout_ms, M, N, K):
    """One GPU as rank 0 of 2; slot buffers, flags and result buffers in pinned host memory so that a CPU thread can be rank 1."""
    from blaze_b200.linear import Linear
    from blaze_b200.quant import Format
    ops, lib, comm, pads, epoch = _setup(timeout_ms)
    lib.blz_gemm_push_rs.argtypes = [VP, VP, VP, VP, ctypes.c_int, ctypes.c_int, ctypes.c_int]
    lib.blz_comm_slots_norm.argtypes = [VP] + [VP] * 9 + [VP, VP, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_float,
                                                         ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, VP]
    per = (M + WORLD - 1) // WORLD
    slots = [torch.zeros(WORLD, per, N, dtype=torch.bfloat16).pin_memory() for _ in range(WORLD)]
    flags = [torch.zeros(16, dtype=torch.int32).pin_memory() for _ in range(WORLD)]
    outs = [torch.zeros(M, N, dtype=torch.bfloat16).pin_memory() for _ in range(WORLD)]
    state = torch.zeros(4, dtype=torch.int32, device="cuda")          # [finished CTAs, epoch]
    g = torch.Generator(device="cuda").manual_seed(12)
    lin = Linear.from_dense(torch.randn(N, K, generator=g, device="cuda") * 0.05, Format.DENSE)
    x = torch.randn(M, K, generator=g, device="cuda").bfloat16()
    lin.keep_alive = epoch          # the communicator holds the raw pointer of its epoch words
    return ops, lib, comm, pads, per, slots, flags, outs, state, lin, x


def _push_and_reduce(ops, lib, comm, per, slots, flags, outs, state, lin, x, residual, w, M, N, blocks):
    arr = lambda ts: (VP * WORLD)(*[VP(t.data_ptr()) for t in ts])      # noqa: E731
    rc = lib.blz_gemm_push_rs(arr(slots), arr(flags), VP(state.data_ptr()), VP(state.data_ptr() + 4), 0, WORLD, per)
    assert rc == 0
    dummy = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    ops.linear(lin, x, out=dummy, wide=False, sk=False)               # rows go to the owners' slots, not to `dummy`
    stream = VP(torch.cuda.current_stream().cuda_stream)
    rc = lib.blz_comm_slots_norm(comm, VP(slots[0].data_ptr()), VP(flags[0].data_ptr()), VP(state.data_ptr() + 4), arr(outs),
                                 VP(0), VP(0), VP(0), VP(0), VP(0), VP(residual.data_ptr()), VP(w.data_ptr()), M, N, per, 1e-6, 0, 0,
                                 blocks, 0, stream)
    assert rc == 0


def test_pushed_reduce_scatter_with_a_cpu_thread_as_the_peer():
    """GEMM epilogue -> peer slot buffers + flag; flag-started reduce + residual + RMSNorm.  The CPU peer reads what the GPU
    pushed for the rows it owns, pushes its own partial rows the other way, and takes part in the closing barrier."""
    from blaze_b200.ops import ref
    M, N, K, blocks = 200, 256, 128, 4
    ops, lib, comm, pads, per, slots, flags, outs, state, lin, x = _push_setup(5000, M, N, K)
    g = torch.Generator().manual_seed(13)
    peer_partial = (torch.randn(M, N, generator=g) * 0.5).bfloat16()
    res_full = (torch.randn(M, N, generator=g) * 0.5).bfloat16()
    w = (1 + 0.1 * torch.randn(N, generator=g)).bfloat16()
    mine = ops.linear(lin, x, wide=False, sk=False).cpu()               # rank 0's partial sums, for the expected values
    total = (mine.float() + peer_partial.float())
    want_h, want_res = ref.rmsnorm(total.bfloat16(), w, 1e-6, res_full)
    failed = []

    def peer():
        deadline = time.monotonic() + 20
        # my partial rows, scattered to their owners' slots at [source rank 1], then my flag on both owners
        slots[0][1, :per] = peer_partial[:per]
        slots[1][1, :M - per] = peer_partial[per:]
        flags[0].numpy()[1] = 1
        flags[1].numpy()[1] = 1
        f = flags[1].numpy()
        while f[0] < 1:                              # rank 0's GEMM has pushed its rows and raised its flag on me
            if time.monotonic() > deadline:
                failed.append("rank 0's flag never arrived")
                return
            time.sleep(0.0005)
        got = slots[1][0, :M - per].float()
        if (got - mine[per:].float()).abs().max().item() != 0.0:
            failed.append("rank 0 pushed wrong rows")
        # reduce my rows and broadcast the normed result, then the closing barrier (exit epoch 2 of every block)
        h = want_h[per:]
        outs[0][per:] = h
        outs[1][per:] = h
        theirs = pads[0].numpy()
        for b in range(blocks):
            theirs[b * SLOTS + 1] = 2

    th = threading.Thread(target=peer)
    th.start()
    residual = res_full[:per].cuda()
    _push_and_reduce(ops, lib, comm, per, slots, flags, outs, state, lin, x, residual, w.cuda(), M, N, blocks)
    torch.cuda.synchronize()
    th.join(timeout=30)
    assert not failed and not th.is_alive(), failed
    assert ops.take_status() == 0
    assert (outs[0].float() - want_h.float()).abs().max().item() < 0.05
    assert torch.equal(outs[0][:per], outs[1][:per])                          # rank 0 broadcast its rows to both
    assert (residual.cpu().float() - want_res[:per].float()).abs().max().item() < 0.05
    lib.blz_comm_destroy(comm)


def test_pushed_reduce_scatter_silent_peer_is_reported():
    """Nobody raises the peer's flag: the owner's bounded wait runs out, the status word says so, nothing is written."""
    M, N, K, blocks = 64, 256, 128, 2
    ops, lib, comm, pads, per, slots, flags, outs, state, lin, x = _push_setup(300, M, N, K)
    residual = torch.zeros(per, N, dtype=torch.bfloat16, device="cuda")
    w = torch.ones(N, dtype=torch.bfloat16, device="cuda")
    t0 = time.monotonic()
    _push_and_reduce(ops, lib, comm, per, slots, flags, outs, state, lin, x, residual, w, M, N, blocks)
    torch.cuda.synchronize()
    assert time.monotonic() - t0 < 10
    assert ops.take_status() == 2
    assert int(flags[1].numpy()[0]) == 1                       # the GEMM still raised its own flag on the peer
    assert int(outs[0].float().abs().sum()) == 0
    x2 = torch.ones(8, device="cuda") * 2
    assert float(x2.sum()) == 16.0 and ops.take_status() == 0
    lib.blz_comm_destroy(comm)
