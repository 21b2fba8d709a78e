"""Bounded device waits and their status words, tested without faulting, trapping or hanging a GPU.

Each test makes a wait run out by leaving unset the thing it waits for, with the wait's limit turned down so that it
runs out in well under a second, then reads the status the kernel recorded and checks that the context still works.
The host-made failures of the plug-in (abort callback, failing allocator) are in test_gpu_plugin.py."""
import ctypes as C
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_peer_wait_gives_up_on_a_rank_that_never_signals_and_names_it():
    """b200_allgather_rows as rank 0 of 2 on one GPU, with nobody playing rank 1: the push lands in both output buffers,
    the wait for rank 1's flag runs into its (shortened) limit, b200_peer_status reports 1 + 1, and after the status is
    cleared a collective of a world of one completes normally on the same context."""
    from cactus_b200._lib import check, lib
    L = lib()
    T, Mg = 8, 64
    src = torch.randn((T, Mg), device="cuda")
    dst = [torch.zeros((T, 2 * Mg), device="cuda") for _ in range(2)]
    flags = [torch.zeros(16, dtype=torch.int32, device="cuda") for _ in range(2)]
    d_arr = (C.c_void_p * 2)(dst[0].data_ptr(), dst[1].data_ptr())
    f_arr = (C.c_void_p * 2)(flags[0].data_ptr(), flags[1].data_ptr())
    st = torch.cuda.current_stream().cuda_stream
    check(L.b200_peer_set_wait_limit(flags[0].data_ptr(), 2000))          # about a millisecond instead of seconds
    check(L.b200_allgather_rows(src.data_ptr(), Mg * 4, T, Mg, 0, 2, d_arr, 2 * Mg * 4, f_arr, st))
    torch.cuda.synchronize()                                              # returns: the wait was bounded
    assert L.b200_peer_status(flags[0].data_ptr()) == 2                   # 1 + the rank that never arrived
    for d in dst:                                                         # the data went out before the wait
        assert torch.equal(d[:, :Mg], src) and not d[:, Mg:].any()
    assert int(flags[1][0]) == 1                                          # rank 0's signal reached rank 1's block
    # the context is usable and the status can be cleared
    check(L.b200_peer_set_wait_limit(flags[0].data_ptr(), 0))
    assert L.b200_peer_status(flags[0].data_ptr()) == 0
    solo = torch.zeros((T, Mg), device="cuda")
    d1 = (C.c_void_p * 1)(solo.data_ptr())
    f1 = (C.c_void_p * 1)(flags[0].data_ptr())
    check(L.b200_allgather_rows(src.data_ptr(), Mg * 4, T, Mg, 0, 1, d1, Mg * 4, f1, st))
    torch.cuda.synchronize()
    assert L.b200_peer_status(flags[0].data_ptr()) == 0 and torch.equal(solo, src)


CHILD = r'''
import sys, numpy as np, torch
sys.path.insert(0, sys.argv[1])
from cactus_b200 import ops
from cactus_b200._lib import lib
from cactus_b200.engine import random_blocks
L = lib()
g = torch.Generator(device="cuda").manual_seed(5)
K, M, N = 1024, 256, 64
w = ops.QWeight.from_blocks(2, K, M, random_blocks(2, M, K, g))
x = torch.randn((N, K), device="cuda", generator=g)
L.b200_kernel_set_wait_limit(64)
before = L.b200_kernel_status()
y = ops.mul_mat(w, x)                      # the tensor-core kernel; its producer copies nothing in this process
torch.cuda.synchronize()                   # returns: every wait was bounded
gave_up = L.b200_kernel_status()
L.b200_kernel_set_wait_limit(0)
cleared = L.b200_kernel_status()
y1 = ops.mul_mat(w, x[:1])                 # one column: the dp4a kernel, on the same context
ref = (x[:1].double() @ ops.dequantize(w).double().t()) if hasattr(ops, "dequantize") else None
torch.cuda.synchronize()
print(before, gave_up, cleared, bool(torch.isfinite(y1).all()), float(y1.abs().max()))
'''


def test_tensor_core_kernel_gives_up_a_wait_that_nothing_completes_and_says_so():
    """The folded-scale tcgen05 kernel with its producer switched off (B200_TCF_DEBUG=32): no stage ever lands, every
    consumer wait runs into the (shortened) limit, the CTAs wait for what they have in flight (nothing), free their
    tensor memory and return; b200_kernel_status is then non-zero, clears, and the context computes another product.
    Runs in a child process because the switches are read once per process."""
    env = dict(os.environ, B200_MMQ_TC="2", B200_TCF_DEBUG="32")
    r = subprocess.run([sys.executable, "-c", CHILD, ROOT], env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr[-2000:]
    before, gave_up, cleared, finite, amax = r.stdout.split()[-5:]
    assert int(before) == 0 and int(gave_up) & 2 and int(cleared) == 0, r.stdout
    assert finite == "True" and float(amax) > 0, r.stdout
