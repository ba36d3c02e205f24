"""CPU: host-side logic - the flash_qla import path, the cu_seqlens caches, the packing / index helpers."""
import pytest
import torch


def test_flash_qla_import_path_resolves_to_this_library():
    # the lines the reference's own callers use (tests/test_gdr.py:18-21, benchmark/bench_gated_delta_rule.py:25-30)
    import flash_qla
    import flashqla_b200 as fq
    from flash_qla import chunk_gated_delta_rule_fwd as fwd
    from flash_qla import chunk_gated_delta_rule_bwd as bwd
    from flash_qla.ops.gated_delta_rule.chunk.arch import is_sm12x  # noqa: F401
    from flash_qla.utils import l2norm, pack, profile  # noqa: F401
    assert fwd is fq.chunk_gated_delta_rule_fwd and bwd is fq.chunk_gated_delta_rule_bwd
    assert flash_qla.chunk_gated_delta_rule is fq.chunk_gated_delta_rule
    assert flash_qla.fused_sigmoid_gating_delta_rule_update is fq.fused_sigmoid_gating_delta_rule_update
    assert flash_qla.flashqla_recurrent_gdn_update is fq.flashqla_recurrent_gdn_update
    assert set(flash_qla.__all__) == {"chunk_gated_delta_rule_fwd", "chunk_gated_delta_rule_bwd", "chunk_gated_delta_rule",
                                      "fused_sigmoid_gating_delta_rule_update", "flashqla_recurrent_gdn_update"}
    with pytest.raises(AttributeError):
        flash_qla.no_such_name
    from flash_qla.ops.gated_delta_rule import chunk_gated_delta_rule as deep
    assert deep is fq.chunk_gated_delta_rule
    x = torch.randn(3, 5, 128)
    assert torch.allclose(l2norm(x).norm(dim=-1), torch.ones(3, 5), atol=1e-4)


def test_seqlen_cache_survives_address_reuse():
    """A serving loop builds a new cu_seqlens per batch; the allocator hands the freed address out again with
    version 0.  The cache must never answer with the previous batch's lengths."""
    from flashqla_b200.utils import host_seqlens
    stale = 0
    for i in range(50):
        a = torch.tensor([0, 10 + i, 30 + 2 * i], dtype=torch.int32)
        assert host_seqlens(a) == [10 + i, 20 + i]
        del a
        b = torch.tensor([0, 7, 9 + i], dtype=torch.int32)
        stale += host_seqlens(b) != [7, 2 + i]
        del b
    assert stale == 0
    c = torch.tensor([0, 4, 8], dtype=torch.int32)
    assert host_seqlens(c) == [4, 4] and host_seqlens(c) == [4, 4]
    c[2] = 9  # in-place edit bumps the version
    assert host_seqlens(c) == [4, 5]
    with pytest.raises(ValueError, match="covers 9 tokens"):
        host_seqlens(c, total_tokens=10)
    with pytest.raises(ValueError, match="non-decreasing"):
        host_seqlens(torch.tensor([0, 5, 3]))


def test_order_cache_is_tied_to_the_tensor():
    from flashqla_b200.utils import longest_first_order
    for i in range(20):
        a = torch.tensor([0, 3, 3 + 50 + i, 60 + i], dtype=torch.int32)
        order = longest_first_order(a, torch.device("cpu"))
        assert order.tolist()[0] == 1
        del a, order
        b = torch.tensor([0, 40 + i, 41 + i, 43 + i], dtype=torch.int32)
        assert longest_first_order(b, torch.device("cpu")).tolist() == [0, 2, 1]
        del b
    assert longest_first_order(torch.tensor([0, 5, 10]), torch.device("cpu")) is None


def test_pack_unpack_and_chunk_index_helpers():
    from flash_qla.utils import (fill_last_chunk_of_g, pack, pad_and_reshape, prepare_chunk_indices,
                                 prepare_chunk_offsets, unpack)
    cu = torch.tensor([0, 5, 5 + 130, 5 + 130 + 64])
    x = torch.arange(199 * 2, dtype=torch.float32).reshape(1, 199, 2)
    padded = unpack(x, cu)
    assert padded.shape == (3, 130, 2) and torch.equal(padded[1, :130], x[0, 5:135]) and padded[0, 5:].abs().sum() == 0
    assert torch.equal(pack(padded, cu), x)
    assert prepare_chunk_offsets(cu, 64).tolist() == [0, 1, 4, 5]
    idx = prepare_chunk_indices(cu, 64)
    assert idx.tolist() == [[0, 0], [1, 0], [1, 1], [1, 2], [2, 0]]
    y = pad_and_reshape(torch.ones(2, 70, 3), 1, 64)
    assert y.shape == (2, 2, 64, 3) and y[:, 1, 6:].sum() == 0
    g = torch.arange(128, dtype=torch.float32).reshape(1, 2, 64).clone()
    fill_last_chunk_of_g(g, 70, None)
    assert g[0, 1, 5] == 69 and (g[0, 1, 6:] == 69).all() and g[0, 0, 63] == 63


def test_chunk_tables_workspace_layout():
    """The host-built chunk tables have the layout the C ABI expects: two int32 exclusive scans, each padded
    to 16 bytes (qla_chunk_fwd_workspace_bytes)."""
    from flashqla_b200 import _cabi
    from flashqla_b200.chunk import chunk_tables_workspace
    cu = [0, 200, 264, 597, 598, 728]
    ws = chunk_tables_workspace(cu, "cpu")["ws"]
    a = _cabi.QlaChunkFwdArgs(num_seqs=5, cu_seqlens=1)
    assert ws.numel() == _cabi.lib().qla_chunk_fwd_workspace_bytes(a)
    t = ws.view(torch.int32)
    assert t[:6].tolist() == [0, 2, 3, 6, 7, 9]
    assert t[ws.numel() // 8:ws.numel() // 8 + 6].tolist() == [0, 4, 5, 11, 12, 15]
