"""Host-side pieces of the decode layer that need no GPU: the rotary table against the rotation the
synthetic keys are made with, and the model shapes against the published parameter counts."""
import torch

from retrievalattention_b200.decode_layer import LLAMA3_8B, QWEN25_7B, QWEN25_72B, cos_sin_cache
from retrievalattention_b200.synthetic import rope_neox


def test_cos_sin_cache_reproduces_the_neox_rotation():
    theta, n = 5e5, 300
    table = cos_sin_cache(n, 128, theta, "cpu")
    assert table.shape == (n, 128) and table.dtype == torch.float32
    x = torch.randn((2, n, 128), generator=torch.Generator().manual_seed(3))
    cos, sin = table[:, :64], table[:, 64:]
    x1, x2 = x[..., :64], x[..., 64:]
    rotated = torch.cat((x1 * cos - x2 * sin, x2 * cos + x1 * sin), dim=-1)
    torch.testing.assert_close(rotated, rope_neox(x, torch.arange(n), theta), rtol=1e-5, atol=1e-5)


def _params(s):
    per_layer = (s.qkv_dim + s.q_heads * s.head_dim) * s.hidden + 3 * s.intermediate * s.hidden + 2 * s.hidden
    return s.layers * per_layer + 2 * s.vocab * s.hidden + s.hidden


def test_model_shapes_match_published_parameter_counts():
    # 8.03 B, 7.6 B (biases of the Qwen projections not counted) and 72.7 B parameters
    assert abs(_params(LLAMA3_8B) / 1e9 - 8.03) < 0.01
    assert abs(_params(QWEN25_7B) / 1e9 - 7.61) < 0.02
    assert abs(_params(QWEN25_72B) / 1e9 - 72.7) < 0.1
    assert LLAMA3_8B.qkv_dim == 6144 and QWEN25_7B.qkv_dim == 4608 and QWEN25_72B.qkv_dim == 10240
