"""How the attention part cuts a step's work for its kernels: decisions made on the host from the step's sizes alone,
so they are checked without a GPU (the number of SMs is given)."""
from types import SimpleNamespace
from unittest import mock

import pytest
import torch

from exl3_server_b200.engine.batch import Workspace, pack_step
from exl3_server_b200.ops import kernels as K
from exl3_server_b200.parts.attention import Attention


def mixer(heads, kv_heads, head_dim, window=0):
    a = Attention.__new__(Attention)
    a.spec = SimpleNamespace(heads=heads, kv_heads=kv_heads, head_dim=head_dim, window=window)
    return a


def tile_keys(lens, size=128):
    return sorted((min(a + size, n) for n in lens for a in range(0, n, size)), reverse=True)


@pytest.fixture(autouse=True)
def gpu_of_148_sms():
    with mock.patch.object(K, "sm_count", lambda device: 148):
        yield


@pytest.mark.parametrize("heads,kv_heads,head_dim", [(36, 36, 64), (16, 2, 64), (32, 8, 128), (32, 2, 128), (6, 3, 80)])
@pytest.mark.parametrize("window", [0, 700])
def test_decode_chunks_are_whole_pages_and_groups_divide_the_heads(heads, kv_heads, head_dim, window):
    a = mixer(heads, kv_heads, head_dim, window)
    for T in (1, 2, 3, 8, 17, 64, 200):
        for keys in (1, 63, 64, 65, 500, 2048, 4096, 16384, 100000):
            split, head_split, in_block = a._decode_split(T, keys, 64, None)
            assert split >= 64 and split % 64 == 0
            assert (heads // kv_heads) % head_split == 0 and (heads // kv_heads) // head_split <= 16
            n = a._chunks(keys, split)
            assert 1 <= n <= K.ATTN_DECODE_MAX_CHUNKS
            assert in_block in (0, 1, 2)
            if in_block:
                assert n <= 4 * in_block                   # a block merges four chunks of an item itself, a cluster eight


def test_decode_choices_at_sizes_that_were_measured():
    two_b = mixer(36, 36, 64)
    assert two_b._decode_split(1, 4096, 64, None) == (512, 1, 2)         # 36 clusters, eight chunks each: 13.6 us
    assert two_b._decode_split(1, 8192, 64, None) == (1024, 1, 2)        # 19.0 us against 23.1 with a block an item
    assert two_b._decode_split(8, 4096, 64, None) == (4096, 1, 0)        # a warp per (token, head), no merge
    assert two_b._decode_split(4, 4096, 64, None) == (1024, 1, 1)        # 144 blocks, four chunks each
    assert two_b._decode_split(8, 16384, 64, None) == (4096, 1, 1)       # two rounds of long items
    assert two_b._decode_split(64, 512, 64, None)[2] == 0                # sixteen rounds of short ones
    eight_b = mixer(32, 2, 128)
    assert eight_b._decode_split(1, 2048, 64, None) == (256, 16, 2)      # every query head a group of its own
    assert eight_b._decode_split(8, 2048, 64, None) == (256, 2, 2)       # 14.4 us against 16.0 with a block an item
    assert eight_b._decode_split(64, 2048, 64, None) == (512, 1, 1)


def test_prompt_kernel_form():
    two_b = mixer(36, 36, 64)
    assert two_b._prefill_variant(tile_keys([2048]), 64, None) == 3      # 576 blocks: two rounds, or one of pairs
    assert two_b._prefill_variant(tile_keys([1536]), 64, None) == 1      # the heaviest tile is the kernel's length
    assert two_b._prefill_variant(tile_keys([1024]), 64, None) == 1      # all blocks at once
    assert two_b._prefill_variant(tile_keys([8192]), 64, None) == 2      # many rounds: four blocks an SM
    assert two_b._prefill_variant(tile_keys([16, 300, 1000, 2048]), 64, None) == 2
    assert two_b._prefill_variant([], 64, None) == 0
    half_b = mixer(16, 2, 64)
    assert half_b._prefill_variant(tile_keys([2048]), 64, None) == 1
    assert half_b._prefill_variant(tile_keys([5000]), 64, None) == 1     # 640 blocks: a few more than four an SM hold
    assert half_b._prefill_variant(tile_keys(list(range(16, 2048, 32))), 64, None) == 2
    # heads of 128 have no four-block kernel; a window bounds what a tile walks
    assert mixer(32, 2, 128)._prefill_variant(tile_keys([2048]), 64, None) == 1
    assert mixer(32, 2, 128)._prefill_variant(tile_keys([8192]), 64, None) in (1, 3)
    assert mixer(36, 36, 64, window=256)._prefill_variant(tile_keys([2048]), 64, None) in (1, 2, 3)
    assert mixer(200, 200, 64)._prefill_variant(tile_keys([4096]), 64, None) in (1, 2, 3)   # more heads than slots


def test_a_step_lists_its_tiles_heaviest_first_with_their_keys():
    ws = Workspace(torch.device("cpu"))
    b = pack_step([0, 1, 2], [0, 100, 640], [list(range(300)), list(range(20)), list(range(130))], [[], [], []],
                  [[[0] * 16] * 3], ws, "cpu")
    seq, q0, n = b.tiles[128]
    keys = b.tile_keys[128]
    assert n == len(keys) == 3 + 1 + 2
    assert keys == sorted(keys, reverse=True)
    starts, counts = [0, 100, 640], [300, 20, 130]
    for i in range(n):
        r, a = int(seq[i]), int(q0[i])
        assert keys[i] == starts[r] + min(a + 128, counts[r])


def test_wide_groups_in_a_block_go_to_two_warps_per_ring():
    eight_b = mixer(32, 2, 128)
    assert eight_b._decode_twins(1, 1) == (2, 2)       # 16 heads: two groups of 8 in one block
    assert eight_b._decode_twins(1, 2) == (2, 2)
    assert eight_b._decode_twins(1, 0) == (1, 1)       # warps sharing all chunks: as it was
    assert eight_b._decode_twins(2, 1) == (2, 1)       # groups of 8 fit one warp's instruction columns
    assert mixer(12, 1, 64)._decode_twins(1, 1) == (2, 2)
    assert mixer(36, 36, 64)._decode_twins(1, 2) == (1, 1)
    assert mixer(22, 2, 64)._decode_twins(1, 1) == (1, 1)      # 11 heads do not halve
