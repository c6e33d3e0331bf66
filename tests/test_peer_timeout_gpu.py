"""A bounded device-side wait that runs out: the fused all-reduce kernel is given a "peer" whose flag nothing
ever sets (a second heap on the same GPU, no second process, no other kernel).  With the wait limit set to a
few milliseconds the kernel returns on its own with status 5 (wait on a peer's flag), the CUDA context stays
usable, and the shard's servicer turns that status into the RuntimeError that fails the batch and stops the
shard.  Nothing faults, traps or hangs."""
import asyncio
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_peer_wait_runs_out_and_the_servicer_fails_the_batch():
    from tgi_b200.ops import cuda as K
    from tgi_b200.server.server import TextGenerationService

    lib = K.load()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    lib.tgi_peer_set_wait_ns.restype = ctypes.c_ulonglong
    lib.tgi_peer_reduce.restype = ctypes.c_int
    heap_bytes = 1 << 20
    heaps = []
    for _ in range(2):
        p = ctypes.c_void_p()
        assert lib.tgi_peer_alloc(ctypes.c_longlong(heap_bytes), ctypes.byref(p)) == 0
        heaps.append(p.value)
    heap_arr = (ctypes.c_void_p * 8)(*(heaps + [0] * 6))
    epoch = torch.zeros(int(lib.tgi_peer_max_blocks()), dtype=torch.int32, device=dev)
    st = K.state(dev)
    assert K.check_status(dev) == 0
    old = lib.tgi_peer_set_wait_ns(ctypes.c_ulonglong(20_000_000))      # 20 ms
    try:
        T, H = 8, 128
        t0 = torch.cuda.Event(enable_timing=True)
        t1 = torch.cuda.Event(enable_timing=True)
        t0.record()
        rc = lib.tgi_peer_reduce(
            heap_arr, ctypes.c_int(0), ctypes.c_int(2), ctypes.c_int(T), ctypes.c_int(H),
            ctypes.c_longlong(0), ctypes.c_longlong(64 << 10), ctypes.c_longlong(128 << 10), ctypes.c_int(8),
            ctypes.c_longlong(256 << 10), K._ptr(epoch), ctypes.c_void_p(0), ctypes.c_void_p(0), ctypes.c_void_p(0),
            ctypes.c_float(0.0), ctypes.c_float(0.0), ctypes.c_int(0), ctypes.c_int(1), K._ptr(st.status),
            ctypes.c_int(0), ctypes.c_longlong(0), ctypes.c_void_p(0), K._stream())
        assert rc == 0
        t1.record()
        torch.cuda.synchronize()                    # returns: the wait gave up by itself
        assert 15.0 < t0.elapsed_time(t1) < 2000.0, "the wait should end after about its 20 ms limit"
    finally:
        lib.tgi_peer_set_wait_ns(ctypes.c_ulonglong(old))

    class _Model:
        device = dev

    service = TextGenerationService(_Model(), cache=None, server_urls=[])
    with pytest.raises(RuntimeError, match="status 5"):
        service._check_kernels()
    # the status word was cleared and the context still works
    assert K.check_status(dev) == 0
    x = torch.randn(64, 256, device=dev, dtype=torch.bfloat16)
    w = torch.randn(128, 256, device=dev, dtype=torch.bfloat16)
    torch.testing.assert_close(K.gemm_bf16(x, w).float(), x.float() @ w.float().t(), atol=0.5, rtol=5e-2)
    for h in heaps:
        lib.tgi_peer_free(ctypes.c_void_p(h))
    assert asyncio.run(service.Health(None, None)) is not None
