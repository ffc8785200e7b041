"""Bookkeeping of the decode caller path (flash_attention_b200/generation.py) that needs no GPU: where
update_kv_cache writes, what it hands back, the limits it enforces, and that InferenceParams carries the
field names the reference's modules read (flash_attn/utils/generation.py:19-36, modules/mha.py:296-322)."""
import dataclasses

import pytest
import torch

from flash_attention_b200.generation import DecodeGraphs, InferenceParams, update_kv_cache


def test_inference_params_has_the_reference_fields_in_order():
    names = [f.name for f in dataclasses.fields(InferenceParams)]
    assert names == ["max_seqlen", "max_batch_size", "seqlen_offset", "batch_size_offset", "key_value_memory_dict",
                     "lengths_per_sample"]
    p = InferenceParams(max_seqlen=16, max_batch_size=2)
    assert p.seqlen_offset == 0 and p.batch_size_offset == 0 and p.key_value_memory_dict == {} and p.lengths_per_sample is None
    assert p.cache_seqlens(2) == 0
    p.lengths_per_sample = torch.tensor([3, 5, 7], dtype=torch.int32)
    assert torch.equal(p.cache_seqlens(2), torch.tensor([3, 5], dtype=torch.int32))
    p.seqlen_offset = 9
    p.reset(32, 4)
    assert (p.max_seqlen, p.max_batch_size, p.seqlen_offset) == (32, 4, 0) and int(p.lengths_per_sample.sum()) == 0


def test_update_kv_cache_writes_in_place_and_returns_the_filled_prefix():
    g = torch.Generator().manual_seed(0)
    p = InferenceParams(max_seqlen=10, max_batch_size=3)
    kv0 = torch.randn(2, 4, 2, 2, 8, generator=g)
    got = update_kv_cache(kv0, p, layer_idx=5)
    cache = p.key_value_memory_dict[5]
    assert cache.shape == (3, 10, 2, 2, 8) and cache.dtype == kv0.dtype  # made on first use, sized by the params
    assert got.shape == (2, 4, 2, 2, 8) and torch.equal(got, kv0)
    assert got.data_ptr() == cache.data_ptr()  # a view of the cache, not a copy
    p.seqlen_offset = 4
    kv1 = torch.randn(2, 1, 2, 2, 8, generator=g)
    got = update_kv_cache(kv1, p, layer_idx=5)
    assert got.shape == (2, 5, 2, 2, 8) and torch.equal(got[:, :4], kv0) and torch.equal(got[:, 4:], kv1)
    # a second group of sequences further down the batch dimension
    p.batch_size_offset, p.seqlen_offset = 2, 0
    kv2 = torch.randn(1, 3, 2, 2, 8, generator=g)
    got = update_kv_cache(kv2, p, layer_idx=5)
    assert torch.equal(cache[2, :3], kv2[0]) and torch.equal(cache[0, :4], kv0[0])
    # limits
    p.batch_size_offset, p.seqlen_offset = 0, 8
    with pytest.raises(ValueError, match="asked to write"):
        update_kv_cache(torch.zeros(2, 3, 2, 2, 8), p, layer_idx=5)
    p.seqlen_offset = 0
    with pytest.raises(ValueError, match="asked to write"):
        update_kv_cache(torch.zeros(4, 1, 2, 2, 8), p, layer_idx=5)


def test_allocate_makes_every_layer_up_front_and_graphs_need_lengths():
    p = InferenceParams(max_seqlen=6, max_batch_size=2).allocate(range(3), nheads_k=2, head_dim=8, dtype=torch.float16,
                                                                 device="cpu")
    assert sorted(p.key_value_memory_dict) == [0, 1, 2]
    assert all(t.shape == (2, 6, 2, 2, 8) and t.dtype == torch.float16 for t in p.key_value_memory_dict.values())
    with pytest.raises(ValueError, match="lengths_per_sample"):
        DecodeGraphs(lambda params, x: x, p)
