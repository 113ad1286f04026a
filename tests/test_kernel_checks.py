"""Host-side index checks of the kernel wrappers (``RONN_KERNEL_CHECKS=1``), on CPU tensors."""
import pytest
import torch

from ronn_b200.ops import checks as C


def _cache(nblocks=6, kv_heads=2, d=8):
    return torch.zeros(nblocks, kv_heads, 16, d)


def test_switch_follows_the_environment(monkeypatch):
    monkeypatch.delenv("RONN_KERNEL_CHECKS", raising=False)
    assert not C.enabled()
    monkeypatch.setenv("RONN_KERNEL_CHECKS", "1")
    assert C.enabled()


def test_paged_attention_arguments():
    kc = _cache()
    q = torch.zeros(3, 4 * 8)
    bt = torch.tensor([[0, 1, 2], [3, 4, 5], [5, 99, 99]], dtype=torch.int32)
    ctx = torch.tensor([48, 17, 16], dtype=torch.int32)
    C.paged_attention(q, kc, bt, ctx, 4, 8, 48)                         # the 99s lie past row 2's context: not read
    with pytest.raises(C.IndexCheckError, match=r"block_tables\[7\] = 99"):
        C.paged_attention(q, kc, bt, torch.tensor([48, 17, 17], dtype=torch.int32), 4, 8, 48)
    with pytest.raises(C.IndexCheckError, match="ctx_len"):
        C.paged_attention(q, kc, bt, torch.tensor([49, 1, 1], dtype=torch.int32), 4, 8, 64)     # table row holds 48 keys
    with pytest.raises(C.IndexCheckError, match="ctx_len"):
        C.paged_attention(q, kc, bt, torch.tensor([-1, 1, 1], dtype=torch.int32), 4, 8, 48)
    with pytest.raises(C.IndexCheckError, match="columns"):
        C.paged_attention(q[:, :16], kc, bt, ctx, 4, 8, 48)
    rows_of = torch.tensor([1, 1, 3], dtype=torch.int32)
    with pytest.raises(C.IndexCheckError, match="bt_row"):
        C.paged_attention(q, kc, bt, ctx, 4, 8, 48, bt_row=rows_of)
    C.paged_attention(q, kc, bt, torch.tensor([16, 16, 16], dtype=torch.int32), 4, 8, 48,
                      bt_row=torch.tensor([1, 1, 0], dtype=torch.int32),
                      append_slots=torch.tensor([-1, 95, 0], dtype=torch.int32), positions=torch.tensor([0, 5, 9]))
    with pytest.raises(C.IndexCheckError, match="append_slots"):
        C.paged_attention(q, kc, bt, ctx, 4, 8, 48, append_slots=torch.tensor([0, 96, 0], dtype=torch.int32))
    with pytest.raises(C.IndexCheckError, match="positions"):
        C.paged_attention(q, kc, bt, ctx, 4, 8, 48, positions=torch.tensor([0, -2, 0]))


def test_append_embedding_and_sequence_arguments():
    kc = _cache()
    qkv = torch.zeros(4, 48)
    C.kv_append(qkv, torch.tensor([0, -1, 95, 7], dtype=torch.int32), kc)
    with pytest.raises(C.IndexCheckError, match=r"slots\[2\] = 96"):
        C.kv_append(qkv, torch.tensor([0, -1, 96, 7], dtype=torch.int32), kc)
    with pytest.raises(C.IndexCheckError, match="entries"):
        C.kv_append(qkv, torch.tensor([0], dtype=torch.int32), kc)
    table, pos_table = torch.zeros(10, 4), torch.zeros(6, 4)
    C.embedding(torch.tensor([0, 9]), table, torch.tensor([5, 0]), pos_table)
    with pytest.raises(C.IndexCheckError, match=r"ids\[1\] = 10"):
        C.embedding(torch.tensor([0, 10]), table)
    with pytest.raises(C.IndexCheckError, match="position table"):
        C.embedding(torch.tensor([0, 1]), table, torch.tensor([6, 0]), pos_table)
    mk = lambda v: torch.tensor(v, dtype=torch.int32)
    C.sequences(100, mk([0, 40]), mk([40, 60]), mk([40, 60]), True)
    with pytest.raises(C.IndexCheckError, match="rows 40..101"):
        C.sequences(100, mk([0, 40]), mk([40, 61]), mk([40, 60]), True)
    with pytest.raises(C.IndexCheckError, match="keys"):
        C.sequences(100, mk([0, 40]), mk([40, 10]), mk([40, 70]), True)
    C.sequences(100, mk([0, 40]), mk([40, 60]), mk([200, 60]), False, table_keys=256)
    with pytest.raises(C.IndexCheckError, match="kv_len"):
        C.sequences(100, mk([0, 40]), mk([40, 60]), mk([300, 60]), False, table_keys=256)
    with pytest.raises(C.IndexCheckError, match="only 50 keys"):
        C.sequences(100, mk([0, 40]), mk([40, 60]), mk([200, 50]), False, table_keys=256)
