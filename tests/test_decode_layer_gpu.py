"""The element-wise kernels of the decode layer (through the C ABI) against plain PyTorch fp32
restatements of the flashinfer calls they replace (model_hub/llama.py:267-275, :304-320), and the
synthetic decoder against a PyTorch restatement of the reference's layer loop
(model_hub/LLM.py:90-126) that drives an identical second cache.

Tolerances: one rounding to the 16-bit type per output element, so 2 ulp of the output's
magnitude for the kernels (rtol 2**-7 for bf16, 2**-10 for fp16); logits of the whole decoder
atol 2e-2 (they are O(1) sums of bf16 products)."""
import pytest
import torch
import torch.nn.functional as F

from retrievalattention_b200.config import generate_config
from retrievalattention_b200.synthetic import make_kv

pytestmark = pytest.mark.gpu

RTOL = {torch.bfloat16: 2.0 ** -7, torch.float16: 2.0 ** -10}


def close(a, b, dtype, atol=1e-3):
    torch.testing.assert_close(a.float(), b.float(), rtol=RTOL[dtype], atol=atol)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("rows,dim", [(4, 4096), (1, 3584), (16, 8192), (3, 8), (2, 16384)])
def test_rmsnorm_and_residual(dtype, rows, dim):
    from retrievalattention_b200.decode_layer import rmsnorm

    g = torch.Generator(device="cuda").manual_seed(rows * 100003 + dim)
    x = torch.randn((rows, dim), generator=g, device="cuda").to(dtype)
    res = torch.randn((rows, dim), generator=g, device="cuda").to(dtype)
    w = (1 + 0.1 * torch.randn((dim,), generator=g, device="cuda")).to(dtype)
    eps = 1e-5

    def ref(h):
        h = h.float()
        return h * torch.rsqrt(h.pow(2).mean(-1, keepdim=True) + eps) * w.float()

    out = torch.empty_like(x)
    rmsnorm(x, w, eps, out)
    close(out, ref(x), dtype)

    res_in = res.clone()
    rmsnorm(x, w, eps, out, residual=res)
    summed = (res_in.float() + x.float()).to(dtype)        # the reference adds in the 16-bit type
    assert torch.equal(res, summed)
    close(out, ref(summed), dtype)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("rows,q_heads,kv_heads", [(4, 32, 8), (8, 28, 4), (1, 1, 1)])
def test_rope_split(dtype, rows, q_heads, kv_heads):
    from retrievalattention_b200.decode_layer import cos_sin_cache, rope_split

    g = torch.Generator(device="cuda").manual_seed(7 + rows)
    heads = q_heads + 2 * kv_heads
    qkv = torch.randn((rows, heads * 128), generator=g, device="cuda").to(dtype)
    cache = cos_sin_cache(4096, 128, 5e5, "cuda")
    pos = torch.randint(0, 4096, (rows,), generator=g, device="cuda", dtype=torch.int64)
    pos[0] = 4095
    q = torch.empty((rows, 1, q_heads, 128), dtype=dtype, device="cuda")
    k = torch.empty((rows, 1, kv_heads, 128), dtype=dtype, device="cuda")
    v = torch.empty((rows, 1, kv_heads, 128), dtype=dtype, device="cuda")
    rope_split(qkv, cache, pos, q, k, v)

    x = qkv.view(rows, heads, 128).float()
    cos, sin = cache[pos][:, None, :64], cache[pos][:, None, 64:]
    x1, x2 = x[..., :64], x[..., 64:]
    rot = torch.cat((x1 * cos - x2 * sin, x2 * cos + x1 * sin), dim=-1)
    close(q.view(rows, q_heads, 128), rot[:, :q_heads], dtype)
    close(k.view(rows, kv_heads, 128), rot[:, q_heads:q_heads + kv_heads], dtype)
    assert torch.equal(v.view(rows, kv_heads, 128), qkv.view(rows, heads, 128)[:, q_heads + kv_heads:])


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("rows,inter", [(4, 14336), (8, 18944), (1, 8), (5, 1000)])
def test_silu_and_mul(dtype, rows, inter):
    from retrievalattention_b200.decode_layer import silu_and_mul

    g = torch.Generator(device="cuda").manual_seed(inter)
    x = (2 * torch.randn((rows, 2 * inter), generator=g, device="cuda")).to(dtype)
    out = torch.empty((rows, inter), dtype=dtype, device="cuda")
    silu_and_mul(x, out)
    close(out, F.silu(x[:, :inter].float()) * x[:, inter:].float(), dtype)


def test_bad_arguments_are_refused():
    from retrievalattention_b200 import _lib

    x = torch.zeros((2, 64), dtype=torch.bfloat16, device="cuda")
    assert _lib.lib.ri_rmsnorm(x.data_ptr(), None, x.data_ptr(), x.data_ptr(), 2, 60, 1e-5, 0, None) == -1
    assert b"dim" in _lib.lib.ri_last_error()
    assert _lib.lib.ri_silu_and_mul(None, x.data_ptr(), 2, 32, 0, None) == -1
    assert _lib.lib.ri_rope_split(x.data_ptr(), None, None, None, None, None, 2, 1, 1, 16, 0, None) == -1


def _make_cache(batch, layers, kv_heads, q_heads, seq_len, max_new):
    from retrievalattention_b200.cache_hub import retroinfer_cache

    cfg = generate_config(seq_len, 0.05, 0.2, n_segments=1)
    mapping = {str(l): "cuda:0" for l in range(layers)}
    cache = retroinfer_cache([0] * batch, layers, batch, seq_len + max_new, kv_heads, q_heads, 128, torch.bfloat16,
                             mapping, max_new, num_gpus=1, model_size=8, **cfg.as_kwargs())
    for b in range(batch):
        for l in range(layers):
            k, v = make_kv(kv_heads, seq_len, 128, seed=31 * l + b, device="cuda")
            cache.prefill_update_kv_cache(None, k, v, l, b)
            cache.sync(l, b)
    cache.prepare_cache()
    return cache


def _reference_step(dec, cache, ids, position):
    """The reference's decode_forward/layer_decode in PyTorch ops on the decoder's weights, fp32
    element-wise arithmetic with the reference's rounding points, attention by ``cache``."""
    s, dt = dec.shape, dec.dtype

    def norm(h, w):
        h = h.float()
        return (h * torch.rsqrt(h.pow(2).mean(-1, keepdim=True) + s.rms_eps) * w.float()).to(dt)

    hidden = dec.embed[ids]
    cs = dec.cos_sin[position]
    cos, sin = cs[:64], cs[64:]
    for ldx, L in enumerate(dec.layers):
        residual = hidden
        qkv = F.linear(norm(hidden, L["norm1"]), L["wqkv"]).view(dec.batch, -1, 128).float()
        x1, x2 = qkv[..., :64], qkv[..., 64:]
        rot = torch.cat((x1 * cos - x2 * sin, x2 * cos + x1 * sin), dim=-1).to(dt)
        q = rot[:, :s.q_heads].reshape(dec.batch, 1, s.q_heads, 128).contiguous()
        k = rot[:, s.q_heads:s.q_heads + s.kv_heads].reshape(dec.batch, 1, s.kv_heads, 128).contiguous()
        v = qkv[:, s.q_heads + s.kv_heads:].to(dt).reshape(dec.batch, 1, s.kv_heads, 128).contiguous()
        cache.decode_update_kv_cache(k, v, ldx)
        attn = cache.compute(q, ldx)
        hidden = residual + F.linear(attn.reshape(dec.batch, -1), L["wo"])
        residual = hidden
        gu = F.linear(norm(hidden, L["norm2"]), L["gate_up"]).float()
        act = (F.silu(gu[:, :s.intermediate]) * gu[:, s.intermediate:]).to(dt)
        hidden = residual + F.linear(act, L["down"])
    return F.linear(norm(hidden, dec.final_norm), dec.lm_head).float()


def test_synthetic_decoder_matches_layer_loop_and_replays_from_a_graph():
    from retrievalattention_b200.decode_layer import ModelShape, SyntheticDecoder

    batch, layers, kv_heads, q_heads, seq_len, max_new = 2, 2, 2, 8, 1024 + 68, 8
    shape = ModelShape(hidden=512, intermediate=1024, vocab=2048, layers=layers, q_heads=q_heads, kv_heads=kv_heads)
    cache_a = _make_cache(batch, layers, kv_heads, q_heads, seq_len, max_new)
    cache_b = _make_cache(batch, layers, kv_heads, q_heads, seq_len, max_new)
    dec = SyntheticDecoder(shape, cache_a, batch, seq_len + max_new, "cuda", seed=5, std=0.05)
    assert int(dec.positions[0]) == seq_len
    dec.input_ids.copy_(torch.tensor([3, 1500], device="cuda"))

    ids = dec.input_ids.clone()
    for step in range(2):                                   # eager steps against the layer loop
        logits = dec.decode_forward()
        ref = _reference_step(dec, cache_b, ids, seq_len + step)
        torch.testing.assert_close(logits, ref, rtol=0, atol=2e-2)
        ids = dec.next_ids.clone()
        assert int(dec.positions[0]) == seq_len + step + 1

    graph = torch.cuda.CUDAGraph()                          # the same step captured, then replayed
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            captured = dec.decode_forward()
    torch.cuda.current_stream().wait_stream(side)
    for step in range(2, 4):
        graph.replay()
        ref = _reference_step(dec, cache_b, ids, seq_len + step)
        torch.testing.assert_close(captured, ref, rtol=0, atol=2e-2)
        ids = dec.next_ids.clone()
    assert int(dec.positions[0]) == seq_len + 4
    assert dec.weight_bytes_per_step() > 0
