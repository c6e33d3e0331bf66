"""Local `rotary` kernel module for the reference (hub: kernels-community/rotary, i.e. flash-attn's
csrc/rotary).  One Triton kernel with the same contract: rotate the pairs (x1, x2) by (cos, sin),
writing out1/out2 (which may alias x1/x2); `conj` rotates backwards."""
import torch
import triton
import triton.language as tl


@triton.jit
def _rotary_kernel(x1_ptr, x2_ptr, cos_ptr, sin_ptr, o1_ptr, o2_ptr, heads, rot,
                   sx_t, sx_h, so_t, so_h, sc_t, CONJ: tl.constexpr, BLOCK: tl.constexpr):
    pid = tl.program_id(0)
    t = pid // heads
    h = pid % heads
    offs = tl.arange(0, BLOCK)
    mask = offs < rot
    x1 = tl.load(x1_ptr + t * sx_t + h * sx_h + offs, mask=mask, other=0.0).to(tl.float32)
    x2 = tl.load(x2_ptr + t * sx_t + h * sx_h + offs, mask=mask, other=0.0).to(tl.float32)
    c = tl.load(cos_ptr + t * sc_t + offs, mask=mask, other=0.0).to(tl.float32)
    s = tl.load(sin_ptr + t * sc_t + offs, mask=mask, other=0.0).to(tl.float32)
    if CONJ:
        s = -s
    tl.store(o1_ptr + t * so_t + h * so_h + offs, x1 * c - x2 * s, mask=mask)
    tl.store(o2_ptr + t * so_t + h * so_h + offs, x1 * s + x2 * c, mask=mask)


def apply_rotary(x1, x2, cos, sin, out1, out2, conj):
    # x1, x2, out1, out2: [tokens, heads, rot] views with a unit inner stride; cos, sin: [tokens, 1, rot]
    tokens, heads, rot = x1.shape
    assert x1.stride(-1) == 1 and x2.stride(-1) == 1 and out1.stride(-1) == 1 and out2.stride(-1) == 1
    assert x1.stride() == x2.stride() and out1.stride() == out2.stride()
    cos = cos.reshape(tokens, -1)
    sin = sin.reshape(tokens, -1)
    assert cos.stride(-1) == 1 and sin.stride() == cos.stride()
    if tokens == 0:
        return
    _rotary_kernel[(tokens * heads,)](
        x1, x2, cos, sin, out1, out2, heads, rot, x1.stride(0), x1.stride(1), out1.stride(0), out1.stride(1),
        cos.stride(0), CONJ=bool(conj), BLOCK=triton.next_power_of_2(rot), num_warps=1)
