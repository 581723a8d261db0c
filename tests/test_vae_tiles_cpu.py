"""Tile batching of the VAE decode (host logic, no GPU): the group sizes of `_tile_groups` and the stitched result of
`tiled_decode_batched` (the scheme of the reference's custom_nodes/rapid_h3/vae_fast.py:321-400)."""
import pytest
import torch

from rapid_h3_b200 import vae_fast


@pytest.mark.parametrize("n", list(range(0, 41)))
@pytest.mark.parametrize("batch", [1, 2, 3, 4, 7, 28, 100])
def test_tile_groups_cover_all_tiles_without_a_lone_tile(n, batch):
    groups = vae_fast._tile_groups(n, batch)
    assert sum(groups) == n
    if n >= 2:
        assert min(groups) >= 2                         # never a single tile beside others
        assert max(groups) - min(groups) <= 1           # as equal as possible
        if batch >= 2:
            assert max(groups) <= max(batch, 3)         # about `batch` per call (pairs and one triple at the low end)
    else:
        assert groups == ([n] if n else [])


def test_tile_groups_examples():
    assert vae_fast._tile_groups(28, 28) == [28]
    assert vae_fast._tile_groups(29, 28) == [15, 14]    # not 28 + 1
    assert vae_fast._tile_groups(7, 1) == [3, 2, 2]     # very low memory: pairs and one triple
    assert vae_fast._tile_groups(1, 4) == [1]


def test_split_tiles():
    starts, lens, ov = vae_fast.split_tiles(100, 40, 8)
    assert starts[0] == 0 and starts[-1] + lens[-1] == 100
    assert all(o >= 8 for o in ov) and len(ov) == len(starts) - 1
    assert vae_fast.split_tiles(32, 40, 8) == ([0], [32], [])


@pytest.mark.parametrize("batch", [1, 2, 5, 100])
@pytest.mark.parametrize("hw", [(9, 13), (4, 4), (16, 7)])
def test_tiled_decode_of_a_local_decoder_equals_the_whole_decode(batch, hw):
    """A decoder whose output pixel depends on its own latent cell only (nearest upsampling times a channel mix)
    gives the same picture tiled or whole: seams are cross-fades of equal values. Also counts the decoder calls."""
    ratio = 8
    g = torch.Generator().manual_seed(3)
    z = torch.randn(1, 4, 3, hw[0], hw[1], generator=g, dtype=torch.float64)
    mix = torch.randn(3, 4, generator=g, dtype=torch.float64)
    calls = []

    def decode(t):
        calls.append(t.shape[0])
        y = torch.einsum("oc,nct...->not...", mix, t)
        return y.repeat_interleave(ratio, -1).repeat_interleave(ratio, -2)

    whole = decode(z)
    calls.clear()
    tiled = vae_fast.tiled_decode_batched(decode, z, ratio, tile=32, overlap=8, batch=batch)
    assert tiled.shape == whole.shape
    assert torch.allclose(tiled, whole, rtol=0, atol=1e-12)
    n_tiles = len(vae_fast.split_tiles(hw[0] * ratio, 32, 8)[0]) * len(vae_fast.split_tiles(hw[1] * ratio, 32, 8)[0])
    assert calls == vae_fast._tile_groups(n_tiles, batch)


def test_blend_is_a_linear_cross_fade():
    a, b = torch.zeros(1, 4, 6), torch.ones(1, 10, 6)
    out = vae_fast.blend(a, b, 4, dim=-2)
    assert torch.allclose(out[0, :4, 0], torch.tensor([0.2, 0.4, 0.6, 0.8])) and torch.equal(out[0, 4:], b[0, 4:])
    with pytest.raises(RuntimeError):
        vae_fast.tiled_decode_batched(lambda t: t, torch.zeros(1, 1, 8, 8), 8, tile=36, overlap=8, batch=2)
