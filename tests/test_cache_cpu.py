"""FgateCache (the generation cache) on CPU tensors: same contents as the concatenating cache it stands in
for (upstream fgate_cache.py:77-116), in-place growth, crop and the batch helpers."""
import pytest
import torch

from forgetting_transformer_b200.cache import FgateCache


def _chunk(g, B, H, T, D):
    return (torch.randn(B, H, T, D, generator=g).bfloat16(), torch.randn(B, H, T, D, generator=g).bfloat16(),
            torch.randn(B, H, T, generator=g))


def test_update_matches_concatenation_and_grows_in_place():
    g = torch.Generator().manual_seed(0)
    B, H, D = 2, 3, 16
    cache = FgateCache(granule=128)
    ref = [None, None]
    ptrs = []
    for T in (100, 1, 1, 27, 1, 200):          # prefill, steps, a second chunk, growth past 128 and 256
        for layer in range(2):
            k, v, lf = _chunk(g, B, H, T, D)
            ko, vo, lo = cache.update(k, v, lf, layer)
            ref[layer] = (k, v, lf) if ref[layer] is None else tuple(
                torch.cat([a, b], dim=d) for a, b, d in zip(ref[layer], (k, v, lf), (2, 2, 2)))
            assert torch.equal(ko, ref[layer][0]) and torch.equal(vo, ref[layer][1]) and torch.equal(lo, ref[layer][2])
            assert ko.stride(-1) == 1 and (ko.stride(2) * ko.element_size()) % 16 == 0
        ptrs.append(cache[0][0].data_ptr())
    assert cache.get_seq_length() == 330 and cache.get_seq_length(1) == 330 and len(cache) == 2
    assert cache._seen_tokens == 330
    assert cache.capacity(0) == 512
    assert ptrs[0] == ptrs[1] == ptrs[2]        # single-token steps write in place: no reallocation
    assert cache.get_seq_length(5) == 0
    with pytest.raises(KeyError):
        cache[2]
    assert [t[0].shape[2] for t in cache] == [330, 330]


def test_log_fgate_rank_is_checked():
    cache = FgateCache()
    k = torch.zeros(1, 1, 4, 8)
    with pytest.raises(AssertionError, match="log_fgate must be"):
        cache.update(k, k, torch.zeros(1, 1, 4, 1), 0)


def test_crop_and_batch_helpers():
    g = torch.Generator().manual_seed(1)
    B, H, D = 4, 2, 8
    cache = FgateCache(granule=128)
    k, v, lf = _chunk(g, B, H, 50, D)
    cache.update(k, v, lf, 0)
    cache.update_shift_cache(torch.arange(B * 16.0).view(B, 16), torch.ones(B, 16), 0)
    with pytest.raises(AssertionError):
        cache.update_shift_cache(torch.zeros(B, 16), torch.zeros(B, 16), 0)     # layer 0 is already registered
    cache.crop(-10)
    assert cache.get_seq_length() == 40 and torch.equal(cache[0][0], k[:, :, :40])
    cache.crop(100)                                                                # longer than the history: no-op
    assert cache.get_seq_length() == 40
    k2, v2, lf2 = _chunk(g, B, H, 3, D)
    ko, _, lo = cache.update(k2, v2, lf2, 0)                                       # overwrites the cropped rows
    assert torch.equal(ko, torch.cat([k[:, :, :40], k2], 2)) and torch.equal(lo, torch.cat([lf[:, :, :40], lf2], 2))
    cache.batch_select_indices(torch.tensor([2, 0]))
    assert torch.equal(cache[0][1], torch.cat([v[:, :, :40], v2], 2)[[2, 0]])
    assert torch.equal(cache.key_shift_cache[0], torch.arange(B * 16.0).view(B, 16)[[2, 0]])
    cache.batch_repeat_interleave(2)
    assert cache[0][0].shape[0] == 4 and torch.equal(cache[0][0][0], cache[0][0][1])
    k3, v3, lf3 = _chunk(g, 4, H, 1, D)
    assert cache.update(k3, v3, lf3, 0)[0].shape == (4, H, 44, D)
    assert len(cache.to_legacy_cache()) == 1 and cache.get_max_length() is None
