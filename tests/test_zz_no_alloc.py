"""GPU test of the allocation-free bf16 GEMM entry point (``tgi_gemm_bf16_static``).

The entry point is called through its exported C symbol with ctypes, twice in a row on each shape,
and compared with the regular entry point (``tgi_gemm_bf16`` through ``ops.cuda.gemm_bf16``), which
takes caller-allocated scratch.  With the same CTA count both run the same kernel on the same split
of the work, so the outputs must be bit-identical.  The file name sorts last on purpose: the test has
to pass both alone and after every other GPU test has used the library in the same process.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

MAX_CTAS = 32        # TGI_STATIC_GEMM_MAX_CTAS
MAX_TILES = 4096     # TGI_STATIC_GEMM_MAX_TILES
ERR_TOO_LARGE = -201


def _lib():
    from tgi_b200.ops import build

    lib = ctypes.CDLL(str(build.LIB_PATH))
    lib.tgi_gemm_bf16_static.restype = ctypes.c_int
    lib.tgi_gemm_bf16_static.argtypes = [ctypes.c_void_p] * 4 + [ctypes.c_int] * 3 + [ctypes.c_void_p]
    lib.tgi_gemm_static_setup.restype = ctypes.c_int
    lib.tgi_gemm_static_status.restype = ctypes.c_int
    lib.tgi_gemm_static_status.argtypes = [ctypes.POINTER(ctypes.c_int), ctypes.c_void_p]
    lib.tgi_gemm_static_strerror.restype = ctypes.c_char_p
    lib.tgi_gemm_static_strerror.argtypes = [ctypes.c_int]
    return lib


def _call(lib, x, w, bias, out):
    stream = torch.cuda.current_stream().cuda_stream
    M, K = x.shape
    N = w.shape[0]
    rc = lib.tgi_gemm_bf16_static(x.data_ptr(), w.data_ptr(), out.data_ptr(),
                                  bias.data_ptr() if bias is not None else None, M, N, K, stream)
    assert rc == 0, lib.tgi_gemm_static_strerror(rc)
    st = ctypes.c_int(-1)
    assert lib.tgi_gemm_static_status(ctypes.byref(st), stream) == 0
    assert st.value == 0, f"kernel status {st.value}"


@pytest.mark.parametrize("M,N,K,with_bias", [
    (256, 1536, 4096, False),    # many K blocks per tile: every tile is split between CTAs
    (48, 1000, 2048, True),      # small-M configuration, ragged N, bias
    (300, 640, 512, False),      # ragged M, few units
])
def test_static_scratch_matches_regular_entry_point(M, N, K, with_bias):
    from tgi_b200.ops import cuda as K_

    lib = _lib()
    torch.cuda.set_device(0)
    assert lib.tgi_gemm_static_setup() == 0
    g = torch.Generator(device="cuda").manual_seed(M * 7 + N)
    x = (torch.randn(M, K, device="cuda", generator=g) * 0.5).to(torch.bfloat16)
    w = (torch.randn(N, K, device="cuda", generator=g) * 0.05).to(torch.bfloat16)
    bias = torch.randn(N, device="cuda", generator=g).to(torch.bfloat16) if with_bias else None

    expect = K_.gemm_bf16(x, w, bias, max_ctas=MAX_CTAS)
    K_.check_status()
    ref = x.float() @ w.float().t()
    if bias is not None:
        ref = ref + bias.float()

    out1 = torch.full((M, N), float("nan"), device="cuda", dtype=torch.bfloat16)
    out2 = torch.full((M, N), float("nan"), device="cuda", dtype=torch.bfloat16)
    _call(lib, x, w, bias, out1)
    _call(lib, x, w, bias, out2)          # second call in a row reuses the same static scratch
    torch.cuda.synchronize()
    assert torch.equal(out1, expect)
    assert torch.equal(out2, expect)
    err = (out1.float() - ref).abs().max().item()
    assert err <= 2e-2 * ref.abs().max().item() + 1e-2


def test_static_scratch_rejects_oversized_problem():
    lib = _lib()
    torch.cuda.set_device(0)
    # M > 128 uses 256 x 128 tiles: N = 128 * (MAX_TILES + 1) columns is one tile too many.  The call
    # is refused before any operand is touched, so tiny placeholder buffers are enough.
    dummy = torch.zeros(16, device="cuda", dtype=torch.bfloat16)
    rc = lib.tgi_gemm_bf16_static(dummy.data_ptr(), dummy.data_ptr(), dummy.data_ptr(), None,
                                  256, 128 * (MAX_TILES + 1), 64, torch.cuda.current_stream().cuda_stream)
    assert rc == ERR_TOO_LARGE
    assert b"limit" in lib.tgi_gemm_static_strerror(rc)
