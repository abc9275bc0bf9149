"""Unit (tile-major) weight layout of the streaming decode GEMV against the GGUF block codecs, on the CPU."""
import pytest
import torch

from ollama_b200.gguf.types import GGMLType
from ollama_b200.models.weights import QWeight
from ollama_b200.ops import sk


@pytest.mark.parametrize("t", [GGMLType.Q4_K, GGMLType.Q6_K])
@pytest.mark.parametrize("shape", [(16, 256), (48, 768), (160, 1024)])
def test_units_decode_to_the_same_weights(t, shape):
    n, k = shape
    w = torch.randn(n, k, generator=torch.Generator().manual_seed(n + k)) * 0.05
    qw = QWeight.from_float("w", w, t)
    u = sk.repack(qw, "cpu")
    assert u.units.shape == (n // 16, k // 256, sk.UNIT_BYTES[u.wtype])
    # Q6_K units are the GGUF bytes reordered; Q4_K units carry the 6-bit scale table unpacked to bytes (+64 per unit)
    assert u.units.numel() == qw.raw.numel() + (64 * u.units.shape[0] * u.units.shape[1] if t == GGMLType.Q4_K else 0)
    assert torch.equal(sk.unit_weights(u), qw.dequant())


def test_interleave_alternates_rows():
    a = QWeight.from_float("a", torch.randn(32, 256), GGMLType.Q4_K)
    b = QWeight.from_float("b", torch.randn(32, 256), GGMLType.Q4_K)
    ab = sk.interleave(a, b).dequant()
    assert torch.equal(ab[0::2], a.dequant()) and torch.equal(ab[1::2], b.dequant())


def test_unsupported_shapes_are_refused():
    q = QWeight.from_float("w", torch.randn(8, 256), GGMLType.Q4_K)
    with pytest.raises(ValueError):
        sk.repack(q, "cpu")
    assert not sk.supported(GGMLType.Q8_0, 16, 256)
