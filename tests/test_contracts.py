"""Host contracts: paged-KV offsets, per-row activation, decode positions and
slots at the 255 / 256 / 257 block boundary.  CPU only.  Modelled on the
reference's tests/test_kv_cache_indexing.py, test_row_contract.py and
test_kv_block_boundary.py."""

import pytest

from dfb_b200 import contracts as K
from dfb_b200.geometry import QWEN3_06B, ModelGeometry


def spec(**kw):
    base = dict(num_layers=28, num_blocks=5, block_size=256, num_kv_heads=8, head_dim=128, dtype_itemsize=2)
    base.update(kw)
    return K.PagedKVCacheSpec(**base)


def test_shape_and_strides():
    s = spec()
    assert s.shape == (2, 28, 5, 256, 8, 128)
    assert (s.head_stride, s.token_stride, s.block_stride, s.layer_stride) == (128, 1024, 262144, 5 * 262144)
    assert s.total_bytes == 2 * 28 * 5 * 262144 * 2


def test_element_offset_formula():
    s = spec()
    table = [3, 1, 4]
    assert s.physical_slot(table, 0) == (3, 0)
    assert s.physical_slot(table, 255) == (3, 255)
    assert s.physical_slot(table, 256) == (1, 0)
    assert s.physical_slot(table, 600) == (4, 88)
    off = s.element_offset(2, table, 257, 5, 17)
    assert off == 2 * s.layer_stride + 1 * s.block_stride + 1 * s.token_stride + 5 * 128 + 17


@pytest.mark.parametrize("bad", [dict(num_layers=0), dict(block_size=0), dict(head_dim=-1)])
def test_spec_rejects_nonpositive(bad):
    with pytest.raises(ValueError):
        spec(**bad)


def test_offset_errors():
    s = spec()
    with pytest.raises(IndexError):
        s.physical_slot([0], -1)
    with pytest.raises(ValueError):
        s.physical_slot([], 0)
    with pytest.raises(IndexError):
        s.physical_slot([0], 256)
    with pytest.raises(ValueError):
        s.physical_slot([-1], 0)       # negative padding would index before the cache
    with pytest.raises(ValueError):
        s.physical_slot([5], 0)
    with pytest.raises(IndexError):
        s.element_offset(28, [0], 0, 0, 0)
    with pytest.raises(IndexError):
        s.element_offset(0, [0], 0, 8, 0)
    with pytest.raises(IndexError):
        s.element_offset(0, [0], 0, 0, 128)


def test_row_active_mask():
    assert K.row_active_mask(None, 3) == [1, 1, 1]
    assert K.row_active_mask([1, 0, True], 3) == [1, 0, 1]
    with pytest.raises(ValueError):
        K.row_active_mask([1, 1], 3)
    with pytest.raises(ValueError):
        K.row_active_mask([0, 0], 2)
    with pytest.raises(ValueError):
        K.row_active_mask(None, 0)


@pytest.mark.parametrize("prompt", [255, 256, 257])
def test_decode_identities_at_block_boundary(prompt):
    bs = 256
    for k in range(3):
        n = prompt + k + 1                       # the sampled token was appended
        assert K.decode_position(n) == prompt + k
        assert K.decode_cache_seqlens(n) == prompt + k
        assert K.decode_cache_len(n) == K.decode_position(n) + 1
        table = list(range(10, 10 + -(-n // bs)))
        slot = K.decode_slot_mapping(table, n, bs)
        assert slot == table[(n - 1) // bs] * bs + (n - 1) % bs


def test_decode_slot_needs_exact_table():
    with pytest.raises(RuntimeError):
        K.decode_slot_mapping([0], 257, 256)      # a block was never appended
    with pytest.raises(RuntimeError):
        K.decode_slot_mapping([0, 1], 256, 256)   # a block was never freed
    with pytest.raises(ValueError):
        K.decode_position(0)


def test_pad_block_table():
    assert K.pad_block_table([3, 4], 4) == [3, 4, 0, 0]
    with pytest.raises(ValueError):
        K.pad_block_table([1, 2, 3], 2)
    assert K.max_pages_per_seq(2048, 256) == 8
    assert K.max_pages_per_seq(1, 256) == 1


def test_geometry_bytes():
    g = QWEN3_06B
    assert g.layer_weight_bytes() == 31_461_888
    assert g.weight_bytes_per_step() == 1_192_099_840
    assert g.kv_bytes_per_token() == 114_688
    assert g.step_bytes([1]) == 1_192_099_840 + 114_688
    assert ModelGeometry(layers=2, vocab=4096).max_pages == 8
