"""The dense comparator (``cache_hub.flash_attn_cache`` + ``attn_hub.decode_full_flash_attn``, the reference's full-attention
baseline, cache_hub/flash_attn_cache.py and attn_hub/flash_attn.py) against fp32 attention over every token, and the
wave-index path beside it on the same prompt — what the comparator is for."""
import pytest
import torch

from retrievalattention_b200.config import generate_config
from retrievalattention_b200.synthetic import make_kv, make_queries

pytestmark = pytest.mark.gpu


def test_dense_decode_matches_fp32_attention_beside_the_wave_index():
    from retrievalattention_b200.attn_hub import decode_full_flash_attn, retroinfer_decode_attn
    from retrievalattention_b200.cache_hub import flash_attn_cache, retroinfer_cache

    batch, layers, kv_heads, q_heads, seq_len, max_new = 2, 2, 2, 8, 2048 + 68, 6
    valid_start = [0, 37]
    mapping = {str(l): "cuda:0" for l in range(layers)}
    dense = flash_attn_cache(valid_start, layers, batch, seq_len + max_new, kv_heads, q_heads, 128, torch.bfloat16,
                             mapping, num_gpus=1, model_size=8)
    cfg = generate_config(seq_len, 0.05, 0.2, n_segments=2)
    wave = retroinfer_cache(valid_start, layers, batch, seq_len + max_new, kv_heads, q_heads, 128, torch.bfloat16,
                            mapping, max_new, num_gpus=1, model_size=8, **cfg.as_kwargs())
    prompts = {}
    for b in range(batch):
        for l in range(layers):
            k, v = make_kv(kv_heads, seq_len, 128, seed=100 * l + b, device="cuda")
            prompts[(l, b)] = (k, v)
            rk, _ = dense.prefill_update_kv_cache(None, k, v, l, b)
            assert rk.shape[1] == seq_len - valid_start[b]
            dense.sync(l, b)
            wave.prefill_update_kv_cache(None, k, v, l, b)
    wave.prepare_cache()
    assert dense.context == seq_len and dense.valid_length.tolist() == [seq_len, seq_len - 37]

    new_rows = {l: [] for l in range(layers)}
    for step in range(3):
        for l in range(layers):
            k_new = make_queries(batch, kv_heads, 128, seed=7000 + 10 * step + l, device="cuda")
            v_new = make_queries(batch, kv_heads, 128, seed=8000 + 10 * step + l, device="cuda")
            q = make_queries(batch, q_heads, 128, seed=9000 + 10 * step + l, device="cuda")
            new_rows[l].append((k_new, v_new))
            kc, vc = dense.decode_update_kv_cache(k_new, v_new, l)
            out = decode_full_flash_attn(q, kc, vc, l, dense)
            wave.decode_update_kv_cache(k_new, v_new, l)
            approx = retroinfer_decode_attn(q, k_new, v_new, l, wave)
            for b in range(batch):
                k, v = prompts[(l, b)]
                ks = torch.cat([k[0, valid_start[b]:]] + [r[0][b] for r in new_rows[l]]).float()      # [tokens, Hk, d]
                vs = torch.cat([v[0, valid_start[b]:]] + [r[1][b] for r in new_rows[l]]).float()
                qb = q[b, 0].float().view(kv_heads, q_heads // kv_heads, 128)
                s = torch.einsum("hgd,thd->hgt", qb, ks) / 128 ** 0.5
                ref = torch.einsum("hgt,thd->hgd", torch.softmax(s, -1), vs).reshape(q_heads, 128)
                err = (out[b, 0].float() - ref).abs()
                assert err.max() <= 2e-2 and err.mean() <= 2e-3, (step, l, b, float(err.max()))
                # the wave index approximates the same quantity (how closely depends on the prompt: these keys are
                # random, the worst case for clustering), so only its sanity is checked here
                assert torch.isfinite(approx[b, 0].float()).all()
    assert dense.context == seq_len + 3 and dense.valid_length.tolist() == [seq_len + 3, seq_len - 37 + 3]
