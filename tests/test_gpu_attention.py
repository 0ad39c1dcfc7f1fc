"""Causal attention against the f16 KV cache, SelfAttention and the whole Block on the GPU, against the oracle's
restatement of the portable arm (src/kernels/kv_attention.rs:155-331) and against their own parts (restating
tests/correctness/model.rs:80-206 in spirit: prefill then decode agree, the block equals its halves)."""
import numpy as np
import pytest
import torch

import oracle as orc
import sme_gemm_b200 as sg
from gpu_util import bits_of, max_rel

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("q_f32", [True, False])
@pytest.mark.parametrize("heads,kv_heads,hd,start,rows", [(4, 4, 64, 0, 1), (8, 2, 32, 5, 3), (6, 3, 128, 17, 40), (2, 1, 256, 100, 1),
                                                         (3, 1, 8, 0, 9), (32, 8, 128, 300, 2)])
def test_attention_matches_the_scalar_statement(heads, kv_heads, hd, start, rows, q_f32):
    rng = np.random.default_rng(heads * 1000 + start + rows)
    cache = sg.KvCache(heads, kv_heads, hd, start + rows + 3)
    k16 = (rng.standard_normal((start + rows, kv_heads * hd)) * 0.7).astype(np.float16)
    v16 = rng.standard_normal((start + rows, kv_heads * hd)).astype(np.float16)
    cache.extend(torch.from_numpy(k16).cuda(), torch.from_numpy(v16).cuda())
    assert cache.len() == start + rows and not cache.is_empty() and cache.row_len() == kv_heads * hd
    q32 = rng.standard_normal((rows, heads * hd)).astype(np.float32)
    if not q_f32:
        q32 = q32.astype(np.float16).astype(np.float32)
    q = torch.from_numpy(q32 if q_f32 else q32.astype(np.float16)).cuda()
    out = torch.zeros((rows, heads * hd), dtype=torch.float32, device="cuda")
    if rows == 1:
        cache.attend(q, out)
    else:
        cache.attend_causal(q, rows, out)
    want = orc.attention_kv_causal(q32, k16.view(np.uint16), v16.view(np.uint16), start, rows, heads, kv_heads, hd, cache.scale())
    # same products and sums in the same order; the device's expf and the order of the probabilities' sum differ
    assert max_rel(out.cpu().numpy(), want) <= 2e-5
    assert sg.last_status() == 0


def test_cache_bookkeeping_and_refusals():
    cache = sg.KvCache(4, 2, 16, 5).with_scale(0.5)
    assert cache.scale() == 0.5 and cache.capacity() == 5 and cache.query_len() == 64 and cache.is_empty()
    row = torch.ones((2, 32), dtype=torch.float16, device="cuda")
    cache.push(row, row)
    cache.extend(row, row)
    assert cache.len() == 4 and tuple(cache.keys().shape) == (4, 32)
    with pytest.raises(AssertionError, match="KvCache full: 4 \\+ 2 rows over capacity 5"):
        cache.extend(row, row)
    cache.truncate(1)
    assert cache.len() == 1
    out = torch.zeros(64, dtype=torch.float32, device="cuda")
    with pytest.raises(AssertionError, match="attend_causal: 3 rows but 1 cached"):
        cache.attend_causal(torch.zeros((3, 64), device="cuda"), 3, torch.zeros((3, 64), device="cuda"))
    cache.clear()
    with pytest.raises(AssertionError, match="needs at least one cached key"):
        cache.attend(torch.zeros(64, device="cuda"), out)
    with pytest.raises(AssertionError, match="head_dim must be a multiple of 8"):
        sg.KvCache(2, 2, 12, 4)
    with pytest.raises(AssertionError, match="positive multiple of kv_heads"):
        sg.KvCache(5, 2, 16, 4)
    L = sg.lib()
    z = torch.zeros(64, device="cuda")
    k = torch.zeros((4, 32), dtype=torch.float16, device="cuda")
    assert L.smeg_attn_kv_causal_dev(out.data_ptr(), z.data_ptr(), 1, 64, k.data_ptr(), k.data_ptr(), 0, 1, 4, 2, 12, 0.5, 0) == -4
    assert L.smeg_attn_kv_causal_dev(out.data_ptr(), z.data_ptr(), 1, 64, k.data_ptr(), k.data_ptr(), 0, 1, 5, 2, 16, 0.5, 0) == -4


def _attention_parts(rng, d, heads, kv_heads, hd):
    w_qkv = (rng.standard_normal(((heads + 2 * kv_heads) * hd, d)) * 0.08).astype(np.float32)
    w_out = (rng.standard_normal((d, heads * hd)) * 0.08).astype(np.float32)
    qkv = sg.Linear.quantize(w_qkv, sg.WeightLayout.OutIn, w_qkv.shape[0], d)
    out = sg.Linear.quantize(w_out, sg.WeightLayout.OutIn, d, heads * hd)
    return sg.SelfAttention.new(qkv, out, heads, kv_heads, hd), w_qkv, w_out


@pytest.mark.parametrize("heads,kv_heads,hd", [(4, 4, 32), (8, 2, 16)])
def test_self_attention_against_the_oracle_chain_and_prefill_then_decode(heads, kv_heads, hd):
    rng = np.random.default_rng(heads + hd)
    d = 128
    attn, w_qkv, w_out = _attention_parts(rng, d, heads, kv_heads, hd)
    m = 21
    x16 = rng.standard_normal((m + 1, d)).astype(np.float16)
    y0 = rng.standard_normal((m + 1, d)).astype(np.float32)
    # prefill m rows, then one more row against the same cache
    cache = attn.cache(64)
    y = torch.from_numpy(y0.copy()).cuda()
    attn.accumulate(torch.from_numpy(x16[:m]).cuda(), cache, y[:m], m)
    attn.accumulate(torch.from_numpy(x16[m:]).cuda(), cache, y[m:], 1)
    assert cache.len() == m + 1
    # all m + 1 rows at once
    cache2 = attn.cache(64)
    y2 = torch.from_numpy(y0.copy()).cuda()
    attn.accumulate(torch.from_numpy(x16).cuda(), cache2, y2, m + 1)
    # (the one-row projection runs on the decode kernel, the block on the GEMM: the cached rows agree to an f16 rounding)
    assert max_rel(cache.keys().float().cpu().numpy(), cache2.keys().float().cpu().numpy()) <= 2e-3
    assert max_rel(cache.values().float().cpu().numpy(), cache2.values().float().cpu().numpy()) <= 2e-3
    assert max_rel(y.cpu().numpy(), y2.cpu().numpy()) <= 2e-3        # decode GEMV and prefill GEMM kernels differ in summation order
    # the oracle's chain: Q4 projection, scalar attention, Q4 projection, residual add
    q_len, kv_len = heads * hd, kv_heads * hd
    qq, qs, _ = orc.q4_quantize(w_qkv, 0, w_qkv.shape[0], d)
    oq, os_, _ = orc.q4_quantize(w_out, 0, d, q_len)
    xb = x16.view(np.uint16)
    qkv_o = orc.f16_bits_to_f32(orc.matmul_q4(xb, qq, qs, None, w_qkv.shape[0], d, 32, m + 1)).reshape(m + 1, -1)
    kb = orc.f32_to_f16_bits(qkv_o[:, q_len:q_len + kv_len])
    vb = orc.f32_to_f16_bits(qkv_o[:, q_len + kv_len:])
    att = orc.attention_kv_causal(qkv_o[:, :q_len], kb, vb, 0, m + 1, heads, kv_heads, hd, cache.scale())
    out_o = orc.f16_bits_to_f32(orc.matmul_q4(orc.f32_to_f16_bits(att), oq, os_, None, d, q_len, 32, m + 1)).reshape(m + 1, d)
    assert max_rel(y2.cpu().numpy(), y0 + out_o) <= 1e-2
    assert sg.last_status() == 0


@pytest.mark.parametrize("rows", [1, 5, 70])
def test_block_equals_its_halves(rows):
    """Block::accumulate (src/block.rs:90-106): norm1 -> attention -> norm2 -> MLP, the same bits as the parts run in turn."""
    rng = np.random.default_rng(rows)
    d, heads, hd, f = 128, 4, 32, 384
    attn, _, _ = _attention_parts(rng, d, heads, heads, hd)
    up = sg.Linear.quantize((rng.standard_normal((f, d)) * 0.05).astype(np.float32), sg.WeightLayout.OutIn, f, d)
    down = sg.Linear.quantize((rng.standard_normal((d, f)) * 0.05).astype(np.float32), sg.WeightLayout.OutIn, d, f)
    n1 = sg.Norm.layer(rng.uniform(0.5, 1.5, d).astype(np.float32), (rng.standard_normal(d) * 0.1).astype(np.float32), 1e-5)
    n2 = sg.Norm.rms(rng.uniform(0.5, 1.5, d).astype(np.float32), 1e-5)
    block = sg.Block.new(n1, attn, n2, sg.Mlp.new(up, sg.Gate.Gelu, down))
    x0 = rng.standard_normal((rows, d)).astype(np.float32)
    cache = block.cache(128)
    warm = torch.from_numpy(rng.standard_normal((3, d)).astype(np.float32)).cuda()
    block.accumulate(warm, cache, 3)                               # three earlier positions
    x = torch.from_numpy(x0.copy()).cuda()
    block.accumulate(x, cache, rows)
    assert cache.len() == 3 + rows
    # the parts, on a cache with the same three positions
    cache2 = block.cache(128)
    cache2.extend(cache.keys()[:3].clone(), cache.values()[:3].clone())
    xp = torch.from_numpy(x0.copy()).cuda()
    h = torch.empty((rows, d), dtype=torch.float16, device="cuda")
    n1.forward(xp, h)
    attn.accumulate(h, cache2, xp, rows)
    n2.forward(xp, h)
    block.mlp.accumulate(h, xp, rows)
    assert torch.equal(x, xp)
    assert torch.isfinite(x).all() and sg.last_status() == 0


def test_two_layer_model_from_a_checkpoint_file(tmp_path):
    """A safetensors file -> Checkpoint -> Blocks (examples/shakespeare/model.rs:84-125 in small): a prompt through both
    layers against the oracle's chain on the same quantised weights, then decode steps against re-running the longer prompt."""
    from sme_gemm_b200.checkpoint import Checkpoint
    from test_checkpoint import write_safetensors
    rng = np.random.default_rng(42)
    d, heads, hd, ff, layers = 64, 2, 32, 256, 2
    tensors = {}
    for i in range(layers):
        p = f"transformer.h.{i}."
        tensors[p + "ln_1.weight"] = ("F32", rng.uniform(0.5, 1.5, d).astype("<f4"))
        tensors[p + "ln_2.weight"] = ("F32", rng.uniform(0.5, 1.5, d).astype("<f4"))
        tensors[p + "attn.c_attn.weight"] = ("F32", (rng.standard_normal((3 * d, d)) * 0.1).astype("<f4"))
        tensors[p + "attn.c_proj.weight"] = ("F32", (rng.standard_normal((d, d)) * 0.1).astype("<f4"))
        tensors[p + "mlp.c_fc.weight"] = ("F32", (rng.standard_normal((ff, d)) * 0.1).astype("<f4"))
        tensors[p + "mlp.c_proj.weight"] = ("F32", (rng.standard_normal((d, ff)) * 0.1).astype("<f4"))
    path = tmp_path / "model.safetensors"
    path.write_bytes(write_safetensors(tensors, {"format": "pt"}))
    ck = Checkpoint.load(path)
    blocks = []
    for i in range(layers):
        p = f"transformer.h.{i}."
        blocks.append(sg.Block.new(ck.norm(p + "ln_1.weight"),
                                   sg.SelfAttention.new(ck.linear(p + "attn.c_attn.weight"), ck.linear(p + "attn.c_proj.weight"), heads, heads, hd),
                                   ck.norm(p + "ln_2.weight"),
                                   sg.Mlp.new(ck.linear(p + "mlp.c_fc.weight"), sg.Gate.Gelu, ck.linear(p + "mlp.c_proj.weight"))))
    rows, extra = 20, 3
    x0 = rng.standard_normal((rows + extra, d)).astype(np.float32)

    def run(n_prefill, n_decode):
        caches = [b.cache(64) for b in blocks]
        x = torch.from_numpy(x0[:n_prefill].copy()).cuda()
        for b, c in zip(blocks, caches):
            b.accumulate(x, c, n_prefill)
        outs = [x]
        for s in range(n_decode):
            xs = torch.from_numpy(x0[n_prefill + s:n_prefill + s + 1].copy()).cuda()
            for b, c in zip(blocks, caches):
                b.accumulate(xs, c, 1)
            outs.append(xs)
        return torch.cat(outs).cpu().numpy()

    got = run(rows, extra)
    whole = run(rows + extra, 0)
    assert max_rel(got, whole) <= 5e-3                                # prefill + decode steps == the longer prompt
    # the oracle's chain for the prompt
    x = x0[:rows].copy()
    scale = float(np.float32(1.0) / np.sqrt(np.float32(hd)))
    for i in range(layers):
        p = f"transformer.h.{i}."
        def lin(name, a_bits, m, nodes=None):
            w, n, k = ck.matrix(p + name)
            q, s, _ = orc.q4_quantize(w, 0, n, k)
            return orc.matmul_q4(a_bits, q, s, None, n, k, 32, m, nodes)
        h16, _ = orc.norm_rows(x, ck.get(p + "ln_1.weight"), None, 1e-5, False)
        qkv = orc.f16_bits_to_f32(lin("attn.c_attn.weight", h16, rows)).reshape(rows, 3 * d)
        att = orc.attention_kv_causal(qkv[:, :d], orc.f32_to_f16_bits(qkv[:, d:2 * d]), orc.f32_to_f16_bits(qkv[:, 2 * d:]), 0, rows,
                                      heads, heads, hd, scale)
        x = x + orc.f16_bits_to_f32(lin("attn.c_proj.weight", orc.f32_to_f16_bits(att), rows)).reshape(rows, d)
        h16, _ = orc.norm_rows(x, ck.get(p + "ln_2.weight"), None, 1e-5, False)
        hid = lin("mlp.c_fc.weight", h16, rows, orc.Nodes([(8, int(sg.Gate.Gelu), 0.0, None, 0)]))
        x = x + orc.f16_bits_to_f32(lin("mlp.c_proj.weight", hid, rows)).reshape(rows, d)
    assert max_rel(got[:rows], x) <= 2e-2
    assert sg.last_status() == 0


@pytest.mark.parametrize("m", [1, 3, 5, 70])
def test_partial_product_is_the_projection_before_its_rounding(m):
    """Linear.partial (one rank's share of a projection split over its input width): the f32 sums whose f16 rounding is
    the projection's output; and a one-rank TpSelfAttention is the block itself."""
    from sme_gemm_b200.tp import TpSelfAttention
    rng = np.random.default_rng(31)
    d, heads, kv_heads, hd = 256, 8, 4, 32
    wo = (rng.standard_normal((d, heads * hd)) * 0.05).astype(np.float32)
    wq = (rng.standard_normal(((heads + 2 * kv_heads) * hd, d)) * 0.05).astype(np.float32)
    out = sg.Linear.quantize(wo, sg.WeightLayout.OutIn, d, heads * hd)
    a = torch.from_numpy(rng.standard_normal((m, heads * hd)).astype(np.float16)).cuda()
    part = torch.zeros((m, d), dtype=torch.float32, device="cuda")
    c = torch.zeros((m, d), dtype=torch.float16, device="cuda")
    out.partial(a, part, m)
    out.forward(a, c, m)
    torch.cuda.synchronize()
    assert max_rel(part.cpu().numpy(), c.float().cpu().numpy()) <= 1e-3
    deq = orc.f16_bits_to_f32(orc.q4_dequant(*orc.q4_quantize(wo, 0, d, heads * hd)[:2], None, d, heads * hd)).reshape(heads * hd, d)
    ref = a.cpu().numpy().astype(np.float64) @ deq.astype(np.float64)
    assert max_rel(part.cpu().numpy(), ref.astype(np.float32)) <= 2e-3
    with pytest.raises(AssertionError, match="plain Q4 weights"):
        sg.Linear.quantize(wo, sg.WeightLayout.OutIn, d, heads * hd, bias=np.zeros(d, np.float16)).partial(a, part, m)
    # world = 1: the tensor-parallel block is the block
    tp = TpSelfAttention.quantize(wq, wo, heads, kv_heads, hd, 0, 1)
    one = sg.SelfAttention(sg.Linear.quantize(wq, sg.WeightLayout.OutIn, wq.shape[0], d), out, heads, kv_heads, hd)
    x = torch.from_numpy(rng.standard_normal((m, d)).astype(np.float16)).cuda()
    y0 = torch.from_numpy(rng.standard_normal((m, d)).astype(np.float32)).cuda()
    y1, y2 = y0.clone(), y0.clone()
    tp.accumulate(x, tp.cache(128), y1, m)
    one.accumulate(x, one.cache(128), y2, m)
    torch.cuda.synchronize()
    assert torch.equal(y1, y2) and sg.last_status() == 0
