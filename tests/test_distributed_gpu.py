"""Distributed engines (CreateDistributedB200MathEngines): one engine per GPU in one process, AllReduce (mean) and
Broadcast through the IMathEngine API over NCCL.  Needs two GPUs; NVLS is switched off for the test."""
import ctypes as C
import os

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_allreduce_mean_and_broadcast_across_two_engines():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    from oracle_lib import ShimmedB200Engine
    if not ShimmedB200Engine.available():
        pytest.skip("libNeoMathEngineB200.so or the shim not built")
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    first = ShimmedB200Engine(device=0)          # loads the libraries; also a plain single engine on device 0
    lib = first.engine_lib
    lib.nb200_create_distributed_math_engines.restype = C.c_int
    lib.nb200_create_distributed_math_engines.argtypes = [C.POINTER(C.c_void_p), C.c_int, C.POINTER(C.c_int), C.c_size_t]
    lib.nb200_engine_all_reduce.restype = C.c_int
    lib.nb200_engine_all_reduce.argtypes = [C.c_void_p, C.c_void_p, C.c_int]
    lib.nb200_engine_broadcast.restype = C.c_int
    lib.nb200_engine_broadcast.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int]
    engines = (C.c_void_p * 2)()
    devices = (C.c_int * 2)(0, 1)
    assert lib.nb200_create_distributed_math_engines(engines, 2, devices, 0) == 0
    try:
        n = 100_003
        host = [np.arange(n, dtype=np.float32) * (r + 1) for r in range(2)]
        dev = [torch.from_numpy(host[r]).to(f"cuda:{r}") for r in range(2)]
        for r in range(2):
            torch.cuda.synchronize(r)
        # AllReduce is collective: each engine's call is made from its own host thread, as NeoML's replicas do
        import threading
        rc = [None, None]

        def reduce(r):
            rc[r] = lib.nb200_engine_all_reduce(engines[r], C.c_void_p(dev[r].data_ptr()), n)
        threads = [threading.Thread(target=reduce, args=(r,)) for r in range(2)]
        [t.start() for t in threads]
        [t.join() for t in threads]
        assert rc == [0, 0]
        want = (host[0] + host[1]) / 2
        for r in range(2):
            torch.cuda.synchronize(r)
            assert np.array_equal(dev[r].cpu().numpy(), want)

        def bcast(r):
            rc[r] = lib.nb200_engine_broadcast(engines[r], C.c_void_p(dev[r].data_ptr()), n, 1)
        dev[1].mul_(3.0)
        torch.cuda.synchronize(1)
        threads = [threading.Thread(target=bcast, args=(r,)) for r in range(2)]
        [t.start() for t in threads]
        [t.join() for t in threads]
        assert rc == [0, 0]
        for r in range(2):
            torch.cuda.synchronize(r)
            assert np.array_equal(dev[r].cpu().numpy(), want * 3)
    finally:
        for r in range(2):
            lib.nb200_destroy_math_engine(engines[r])
        first.close()
