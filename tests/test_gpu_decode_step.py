"""The decode step around the linears: the fused producers (residual + RMSNorm + rotation, SiLU(gate) * up + rotation, plain
rotation) feed exl3_linear_prerotated the same fragments a stand-alone exl3_linear builds for itself -- so results must be
equal bit for bit -- and a small two-layer `DecodeStep` (RoPE, KV cache, attention, residuals) agrees with a float64
restatement built on the oracle's decoder."""
from __future__ import annotations

import numpy as np
import pytest
import torch

from oracle import exl3_oracle as orc
from trellis_serve_b200.kernels import linear as lin
from trellis_serve_b200.runtime.decode_step import DecodeStep, ModelShape
from trellis_serve_b200.runtime.layerset import random_packed, random_signs

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")


def _group(k, ns, K, seed):
    gen = torch.Generator(device=DEV)
    gen.manual_seed(seed)
    packed = torch.cat([random_packed(k, n, K, gen, DEV) for n in ns])
    suh = random_signs(k, gen, DEV, len(ns))
    svh = (random_signs(sum(ns), gen, DEV).view(-1).float() / 32).half()
    ends = [sum(ns[:i + 1]) for i in range(len(ns) - 1)]
    ws = torch.zeros(lin.workspace_bytes(16, k, sum(ns), len(ns)), dtype=torch.uint8, device=DEV)
    return packed, suh, svh, ends, ws, gen


@pytest.mark.parametrize("rows,dtype,K,cb", [(1, torch.float16, 3, 0), (2, torch.bfloat16, 4, 1), (5, torch.float16, 3, 2), (16, torch.bfloat16, 5, 0)])
def test_fused_producers_give_the_bits_of_the_stand_alone_linear(rows, dtype, K, cb):
    k, ns = 1024, [640, 384]
    packed, suh, svh, ends, ws, gen = _group(k, ns, K, 11 * rows + K)
    x = torch.randn((rows, k), device=DEV, generator=gen).to(dtype)
    out = torch.empty((rows, sum(ns)), dtype=dtype, device=DEV)
    # plain rotation ahead of the linear
    lin.rotate_fragments(x, suh, cb, ws)
    lin.run_prerotated(rows, packed, svh, ends, cb, out, ws)
    assert torch.equal(out.view(torch.int16), lin.run(x, packed, suh, svh, ends, cb).view(torch.int16))
    # residual add + RMSNorm + rotation
    res0 = torch.randn((rows, k), device=DEV, generator=gen).to(dtype)
    weight = (1.0 + 0.1 * torch.randn(k, device=DEV, generator=gen)).to(dtype)
    residual, normed = res0.clone(), torch.empty_like(x)
    lin.rmsnorm_rotate(x, residual, weight, 1e-6, suh, cb, ws, normed=normed)
    lin.run_prerotated(rows, packed, svh, ends, cb, out, ws)
    torch.cuda.synchronize()
    assert torch.equal(residual, (x.float() + res0.float()).to(dtype))
    want = torch.nn.functional.rms_norm(residual.float(), (k,), weight.float(), 1e-6)
    assert float((normed.float() - want).abs().max()) <= (2e-2 if dtype == torch.bfloat16 else 3e-3)
    assert torch.equal(out.view(torch.int16), lin.run(normed, packed, suh, svh, ends, cb).view(torch.int16))
    # no residual: the input itself is normalised and stays untouched
    x_before = x.clone()
    lin.rmsnorm_rotate(x, None, weight, 1e-6, suh, cb, ws, normed=normed)
    assert torch.equal(x, x_before)
    want = torch.nn.functional.rms_norm(x.float(), (k,), weight.float(), 1e-6)
    assert float((normed.float() - want).abs().max()) <= (2e-2 if dtype == torch.bfloat16 else 3e-3)
    lin.device_error(DEV)


@pytest.mark.parametrize("rows,dtype,K,cb", [(1, torch.float16, 3, 0), (2, torch.bfloat16, 4, 1), (2, torch.float16, 3, 2), (5, torch.bfloat16, 3, 0)])
def test_normalisation_inside_the_linear(rows, dtype, K, cb):
    """exl3_rmsnorm_linear against exl3_rmsnorm_rotate + exl3_linear_prerotated: the new residual stream is the same bits; the
    outputs agree to the last bit of the normalisation factor (the mean square is added in another order), i.e. to an ulp of a few
    activations ahead of the rotation -- far inside the 2e-3 of the linear itself.  Five rows take the normalisation kernel."""
    k, ns = 1024, [640, 384]
    packed, suh, svh, ends, ws, gen = _group(k, ns, K, 7 * rows + K)
    x = torch.randn((rows, k), device=DEV, generator=gen).to(dtype)
    res0 = torch.randn((rows, k), device=DEV, generator=gen).to(dtype)
    weight = (1.0 + 0.1 * torch.randn(k, device=DEV, generator=gen)).to(dtype)
    want, got = torch.empty((rows, sum(ns)), dtype=dtype, device=DEV), torch.empty((rows, sum(ns)), dtype=dtype, device=DEV)
    residual = res0.clone()
    lin.rmsnorm_rotate(x, residual, weight, 1e-6, suh, cb, ws)
    lin.run_prerotated(rows, packed, svh, ends, cb, want, ws)
    res_out = torch.full_like(res0, float("nan"))
    lin.run_rmsnorm(x, res0, res_out, weight, 1e-6, packed, suh, svh, ends, cb, got, ws)
    torch.cuda.synchronize()
    assert torch.equal(res_out, residual)
    scale = float(want.float().pow(2).mean().sqrt())
    assert float((got.float() - want.float()).abs().max()) <= 2e-3 * scale
    # no residual: x itself is normalised
    lin.rmsnorm_rotate(x, None, weight, 1e-6, suh, cb, ws)
    lin.run_prerotated(rows, packed, svh, ends, cb, want, ws)
    lin.run_rmsnorm(x, None, None, weight, 1e-6, packed, suh, svh, ends, cb, got, ws)
    assert float((got.float() - want.float()).abs().max()) <= 2e-3 * scale
    lin.device_error(DEV)


@pytest.mark.parametrize("rows,dtype,glu", [(1, torch.float16, False), (2, torch.bfloat16, True), (1, torch.bfloat16, True), (2, torch.float16, False),
                                            (5, torch.float16, True), (6, torch.bfloat16, False)])
def test_residual_stream_in_the_epilogue_and_its_consumer(rows, dtype, glu):
    """A row-parallel end of a block (o or down) with the residual epilogue: the new stream is exactly round(y + z) for the y the
    plain call stores, its sums of squares per 128 columns are those of the stored stream, y may be left out; the consumer
    (`run_normed`) on that stream agrees with the normalisation kernel + linear to the last bit of the normalisation factor.
    Five and six rows take the kernels around a plain GEMV."""
    k, n, K, cb = 768, 1024, 3, 0
    packed, suh, svh, ends, ws, gen = _group(k, [n], K, 13 * rows + glu)
    z = torch.randn((rows, n), device=DEV, generator=gen).to(dtype)
    y = torch.empty((rows, n), dtype=dtype, device=DEV)
    z2, ssq = torch.full_like(z, float("nan")), torch.full((rows, n // 128), float("nan"), dtype=torch.float32, device=DEV)
    if glu:
        gu = torch.randn((rows, 2 * k), device=DEV, generator=gen).to(dtype)
        lin.run_glu(gu, packed, suh.view(-1), svh, cb, y, ws)
        plain = y.clone()
        lin.run_glu(gu, packed, suh.view(-1), svh, cb, y, ws, residual=(z, z2, ssq))
    else:
        x = torch.randn((rows, k), device=DEV, generator=gen).to(dtype)
        lin.rotate_fragments(x, suh, cb, ws)
        lin.run_prerotated(rows, packed, svh, ends, cb, y, ws)
        plain = y.clone()
        lin.rotate_fragments(x, suh, cb, ws)
        lin.run_prerotated(rows, packed, svh, ends, cb, y, ws, residual=(z, z2, ssq))
    torch.cuda.synchronize()
    assert torch.equal(y, plain)
    want = (plain.float() + z.float()).to(dtype)
    assert torch.equal(z2, want)
    want_ssq = want.float().view(rows, n // 128, 128).pow(2).sum(-1)
    assert float(((ssq - want_ssq).abs() / want_ssq).max()) <= 1e-5
    if rows <= 2:                                      # y is optional when the epilogue carries the stream
        z3, ssq3 = torch.full_like(z, float("nan")), torch.zeros_like(ssq)
        if glu:
            lin.run_glu(gu, packed, suh.view(-1), svh, cb, None, ws, residual=(z, z3, ssq3))
        else:
            lin.rotate_fragments(x, suh, cb, ws)
            lin.run_prerotated(rows, packed, svh, ends, cb, None, ws, residual=(z, z3, ssq3))
        assert torch.equal(z3, z2) and torch.equal(ssq3, ssq)
    # the consumer of that stream: a fused group of the stream's width
    packed2, suh2, svh2, ends2, ws2, gen2 = _group(n, [640, 384], 4, 5 + rows)
    weight = (1.0 + 0.1 * torch.randn(n, device=DEV, generator=gen2)).to(dtype)
    got, ref = torch.empty((rows, 1024), dtype=dtype, device=DEV), torch.empty((rows, 1024), dtype=dtype, device=DEV)
    lin.run_normed(z2, ssq, weight, 1e-6, packed2, suh2, svh2, ends2, 1, got, ws2)
    lin.rmsnorm_rotate(z2, None, weight, 1e-6, suh2, 1, ws2)
    lin.run_prerotated(rows, packed2, svh2, ends2, 1, ref, ws2)
    torch.cuda.synchronize()
    scale = float(ref.float().pow(2).mean().sqrt())
    assert float((got.float() - ref.float()).abs().max()) <= 2e-3 * scale
    lin.device_error(DEV)


@pytest.mark.parametrize("rows,dtype", [(1, torch.float16), (2, torch.bfloat16), (7, torch.float16)])
def test_silu_mul_rotation_feeds_the_down_projection(rows, dtype):
    inter, n, K, cb = 768, 512, 3, 0
    packed, suh, svh, ends, ws, gen = _group(inter, [n], K, 90 + rows)
    gu = torch.randn((rows, 2 * inter), device=DEV, generator=gen).to(dtype)
    act, out = torch.empty((rows, inter), dtype=dtype, device=DEV), torch.empty((rows, n), dtype=dtype, device=DEV)
    lin.silu_mul_rotate(gu, suh, cb, ws, act=act)
    lin.run_prerotated(rows, packed, svh, ends, cb, out, ws)
    want = torch.nn.functional.silu(gu[:, :inter].float()) * gu[:, inter:].float()
    assert float((act.float() - want).abs().max()) <= (3e-2 if dtype == torch.bfloat16 else 4e-3)
    assert torch.equal(out.view(torch.int16), lin.run(act, packed, suh, svh, ends, cb).view(torch.int16))
    # the same projection fed straight from gate | up: the activation inside the GEMV's own rotation (up to two rows) or the
    # activation kernel ahead of it (more rows) -- the same bits either way
    out2 = torch.full_like(out, float("nan"))
    lin.run_glu(gu, packed, suh.view(-1), svh, cb, out2, ws)
    assert torch.equal(out2.view(torch.int16), out.view(torch.int16))
    lin.device_error(DEV)


def _ref_linear(x64, packed, suh, svh, K, cb, col0, n):
    """float64 forward of columns [col0, col0 + n) of a fused group on the oracle's decoded weights."""
    tr = lin.unprepare_matrix(packed[col0 // 128:(col0 + n) // 128].contiguous()).cpu().numpy().view(np.uint16)
    return orc.np_linear_forward(x64, tr, suh.cpu().numpy().astype(np.float64), svh[col0:col0 + n].cpu().numpy().astype(np.float64), K, cb,
                                 np.float64, reconstruct=orc.c_reconstruct)


def test_library_attention_equals_the_stock_path():
    """RoPE + cache append + split-KV attention + merge against torch's rotary arithmetic and scaled_dot_product_attention on
    the same q|k|v and cache: grouped queries (5 per KV head), a context that spans several 128-position chunks and ends
    inside one, fp16 and bf16."""
    for dtype, ctx in ((torch.float16, 300), (torch.bfloat16, 127)):
        shape = ModelShape(hidden=256, q_heads=10, kv_heads=2, head_dim=128, ffn=512, layers=1)
        a = DecodeStep(shape, 3, 0, ctx, rows=2, device=DEV, seed=5, dtype=dtype, attention="library")
        b = DecodeStep(shape, 3, 0, ctx, rows=2, device=DEV, seed=5, dtype=dtype, attention="torch")
        gen = torch.Generator(device=DEV)
        gen.manual_seed(9)
        qkv = torch.randn(a.qkv.shape, device=DEV, generator=gen).to(dtype)
        b.kv.copy_(a.kv)
        a.qkv.copy_(qkv)
        b.qkv.copy_(qkv)
        a._attention(0)
        b._attention(0)
        torch.cuda.synchronize()
        tol = 2e-2 if dtype == torch.bfloat16 else 3e-3
        assert float((a.attn.float() - b.attn.float()).abs().max()) <= tol
        assert float((a.kv[0].float() - b.kv[0].float()).abs().max()) <= tol          # the appended key (rotated) and value


@pytest.mark.parametrize("attention", ["library", "torch"])
def test_two_layer_decode_step_against_a_float64_restatement(attention):
    shape = ModelShape(hidden=256, q_heads=2, kv_heads=1, head_dim=128, ffn=512, layers=2)
    K, cb, ctx = 4, 1, 24
    step = DecodeStep(shape, K, cb, ctx, rows=1, device=DEV, seed=77, attention=attention)
    gen = torch.Generator(device=DEV)
    gen.manual_seed(5)
    step.h_in.copy_(torch.randn((1, shape.hidden), device=DEV, generator=gen).half())
    kv0 = step.kv.clone()
    eager = step.step().clone()
    step.kv.copy_(kv0)
    step.capture()
    step.kv.copy_(kv0)
    replayed = step.replay().clone()
    torch.cuda.synchronize()
    lin.device_error(DEV)
    assert torch.equal(eager, replayed)

    def rms(v, w):
        return v / np.sqrt((v ** 2).mean(-1, keepdims=True) + shape.eps) * w

    def rope(t, heads):
        x = t.reshape(1, heads, shape.head_dim)
        c, s = step.cos.double().cpu().numpy(), step.sin.double().cpu().numpy()
        x1, x2 = x[..., :64], x[..., 64:]
        return np.concatenate([x1 * c - x2 * s, x2 * c + x1 * s], -1)
    h = step.h_in.double().cpu().numpy()
    residual = np.zeros_like(h)
    q, kv, f = shape.q_out, shape.kv_out, shape.ffn
    for i, (qkv, o, gu, down, norms) in enumerate(step.layers):
        nw = norms.double().cpu().numpy()
        residual = residual + h
        a = rms(residual, nw[0])
        y = np.concatenate([_ref_linear(a, qkv.packed, qkv.suh[j], qkv.svh, K, cb, c0, w) for j, (c0, w) in enumerate([(0, q), (q, kv), (q + kv, kv)])], 1)
        qh, kh, vh = rope(y[:, :q], shape.q_heads), rope(y[:, q:q + kv], shape.kv_heads), y[:, q + kv:].reshape(1, 1, 128)
        kc, vc = kv0[i, 0, 0].double().cpu().numpy().copy(), kv0[i, 1, 0].double().cpu().numpy().copy()      # [kv heads, ctx + 1, d]
        kc[:, ctx], vc[:, ctx] = kh[0], vh[0]
        att = np.zeros((1, shape.q_heads, 128))
        for hd in range(shape.q_heads):
            sc = kc[0] @ qh[0, hd] / np.sqrt(128.0)
            p = np.exp(sc - sc.max())
            att[0, hd] = (p / p.sum()) @ vc[0]
        oo = _ref_linear(att.reshape(1, q), o.packed, o.suh[0], o.svh, K, cb, 0, shape.hidden)
        residual = residual + oo
        a = rms(residual, nw[1])
        g = np.concatenate([_ref_linear(a, gu.packed, gu.suh[j], gu.svh, K, cb, j * f, f) for j in range(2)], 1)
        act = g[:, :f] / (1 + np.exp(-g[:, :f])) * g[:, f:]
        h = _ref_linear(act, down.packed, down.suh[0], down.svh, K, cb, 0, shape.hidden)
    want = rms(residual + h, step.final_norm.double().cpu().numpy())
    got = eager.double().cpu().numpy()
    assert np.isfinite(got).all()
    assert orc.rel_norm(got, want) <= 1.5e-2, orc.rel_norm(got, want)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("q_heads,kv_heads,pos", [(10, 2, 300), (8, 8, 127), (16, 2, 128), (4, 1, 0)])
def test_rope_inside_the_attention_kernel_gives_the_bits_of_the_separate_launch(dtype, q_heads, kv_heads, pos):
    """exl3_rope_decode_attention == exl3_rope_append followed by exl3_decode_attention: output, appended cache slot and the o
    projection's rotated fragments, bit for bit; positions at the start, at the end of a 128-position chunk and at the start of
    the next one."""
    import ctypes
    import math
    from trellis_serve_b200 import _lib
    from trellis_serve_b200.kernels import linear as lin
    lib, rows, t_max = _lib.load(), 2, 384
    _lib.init_device(0)
    gen = torch.Generator(device=DEV)
    gen.manual_seed(pos + q_heads)
    heads = q_heads + 2 * kv_heads
    qkv = torch.randn((rows, heads * 128), device=DEV, generator=gen).to(dtype)
    cache = torch.randn((2, rows, kv_heads, t_max, 128), device=DEV, generator=gen).to(dtype)
    inv = 1.0 / (10000.0 ** (torch.arange(0, 64, device=DEV, dtype=torch.float32) / 64))
    ang = torch.arange(t_max, device=DEV, dtype=torch.float32)[:, None] * inv[None]
    cos_t, sin_t = ang.cos().contiguous(), ang.sin().contiguous()
    position = torch.tensor([pos], dtype=torch.int32, device=DEV)
    suh = (torch.randint(0, 2, (q_heads * 128,), device=DEV, generator=gen) * 2 - 1).half()
    scratch = torch.zeros(int(lib.exl3_attention_scratch_bytes(rows, q_heads, kv_heads, t_max)), dtype=torch.uint8, device=DEV)
    need = int(lib.exl3_linear_workspace_bytes(rows, q_heads * 128, 256, 1))
    p, st, code, scale = lin._ptr, lin._stream(torch.device(DEV)), lin._dtype_code(qkv), 1.0 / math.sqrt(128)
    results = []
    for fused in (False, True):
        q2, c2 = qkv.clone(), cache.clone()
        out = torch.empty((rows, q_heads * 128), dtype=dtype, device=DEV)
        ws = torch.zeros(need, dtype=torch.uint8, device=DEV)
        if fused:
            _lib.check(lib.exl3_rope_decode_attention(p(q2), code, rows, q_heads, kv_heads, 128, p(cos_t), p(sin_t), p(c2[0]), p(c2[1]), t_max,
                                                      p(position), scale, p(scratch), scratch.numel(), p(out), p(suh), 0, p(ws), ws.numel(), st),
                       "exl3_rope_decode_attention")
        else:
            _lib.check(lib.exl3_rope_append(p(q2), code, rows, q_heads, kv_heads, 128, p(cos_t), p(sin_t), p(c2[0]), p(c2[1]), t_max,
                                            p(position), st), "exl3_rope_append")
            _lib.check(lib.exl3_decode_attention(p(q2), code, rows, q_heads, kv_heads, 128, p(c2[0]), p(c2[1]), t_max, p(position), scale,
                                                 p(scratch), scratch.numel(), p(out), p(suh), 0, p(ws), ws.numel(), st), "exl3_decode_attention")
        torch.cuda.synchronize()
        results.append((out, c2, ws))
    assert torch.equal(results[0][0], results[1][0])
    assert torch.equal(results[0][1], results[1][1])
    assert torch.equal(results[0][2], results[1][2])
    assert torch.isfinite(results[1][0].float()).all()
