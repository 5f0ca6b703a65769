"""Peer buffers and the flag barrier of the tensor-parallel layer, as far as one GPU can show them.

The barrier's wait is bounded: a rank that never signals costs the others one timeout and a status
word, not a hang. The test below lets the wait run out on purpose -- a flag array nobody writes stands
in for the missing rank -- and checks the status; nothing faults and the context stays usable."""
import pytest
import torch

from bsipytorch_b200 import bsi_ops

pytestmark = pytest.mark.gpu
DEV = "cuda"


def test_peer_alloc_gives_a_zeroed_buffer_and_a_handle():
    buf, handle = bsi_ops.peer_alloc(4096)
    assert buf.dtype == torch.uint8 and buf.numel() == 4096 and buf.is_cuda
    assert isinstance(handle, bytes) and len(handle) == 64
    assert not buf.any()
    buf[:16] = 7
    assert int(buf.sum()) == 112


def test_barrier_of_one_rank_passes_and_counts():
    buf, _ = bsi_ops.peer_alloc(256)
    for expect in (1, 2, 3):
        bsi_ops.peer_barrier([buf.data_ptr()], 0, 100)
        torch.cuda.synchronize()
        flags = buf[:8].view(torch.int32)
        assert int(flags[0]) == expect and int(flags[1]) == expect     # own slot and the epoch counter
    assert bsi_ops.device_status() == 0


def test_barrier_gives_up_on_a_rank_that_never_arrives():
    mine, _ = bsi_ops.peer_alloc(256)
    silent, _ = bsi_ops.peer_alloc(256)           # stands in for rank 1: nobody ever writes its slot in `mine`
    bsi_ops.peer_barrier([mine.data_ptr(), silent.data_ptr()], 0, 50)
    torch.cuda.synchronize()
    assert bsi_ops.device_status() == 64 + 1       # gave up waiting for rank 1
    assert bsi_ops.device_status() == 0            # reading clears the word
    assert int(silent[:4].view(torch.int32)[0]) == 1   # the signal to the other rank was sent before the wait
    # the context is intact: a later kernel runs
    x = torch.randn(4, 256, device=DEV)
    q8 = torch.empty(4, 256, dtype=torch.int8, device=DEV)
    sc = torch.empty(4, 1, device=DEV)
    bsi_ops.pack_queries_into(x, q8, sc, 2)
    torch.cuda.synchronize()
    assert q8.any()


def test_pack_multi_writes_every_destination():
    g = torch.Generator().manual_seed(3)
    x = torch.randn(64, 512, generator=g).half().to(DEV)
    want_q8 = torch.empty(64, 512, dtype=torch.int8, device=DEV)
    want_sc = torch.empty(64, 2, device=DEV)
    bsi_ops.pack_queries_into(x, want_q8, want_sc, 2)
    wide = torch.full((3, 64, 1024), 99, dtype=torch.int8, device=DEV)       # destinations: column block 512.. of each
    scs = torch.full((3, 64, 4), -1.0, device=DEV)
    bsi_ops.pack_queries_multi(x, [wide[i].data_ptr() + 512 for i in range(3)], 1024,
                               [scs[i].data_ptr() + 8 for i in range(3)], 4, 2)
    for i in range(3):
        assert torch.equal(wide[i][:, 512:], want_q8) and (wide[i][:, :512] == 99).all()
        assert torch.equal(scs[i][:, 2:], want_sc) and (scs[i][:, :2] == -1.0).all()


def test_linear_scatter_deals_rows_to_their_owners():
    g = torch.Generator().manual_seed(4)
    x = torch.randn(128, 512, generator=g).half().to(DEV)
    w = (torch.randn(256, 512, generator=g) * 0.05).to(DEV)
    bias = torch.randn(256, generator=g).to(DEV)
    cap = bsi_ops.build_bsi_keys_cuda(w, 2, 0.5)[0]
    q8 = torch.empty(128, 512, dtype=torch.int8, device=DEV)
    sc = torch.empty(128, 2, device=DEV)
    bsi_ops.pack_queries_into(x, q8, sc, 2)
    want = bsi_ops.linear_from_packed(q8, sc, cap, bias, 2, torch.float16, False)
    owners = torch.full((4, 32, 512), 7.0, dtype=torch.float16, device=DEV)   # 4 owners x 32 rows, columns 256.. are ours
    bsi_ops.linear_from_packed_scatter(q8, sc, cap, bias, 2, torch.float16, False,
                                       [owners[i].data_ptr() + 256 * 2 for i in range(4)], 32, 512)
    for i in range(4):
        assert torch.equal(owners[i][:, 256:], want[32 * i:32 * (i + 1)])
        assert (owners[i][:, :256] == 7.0).all()
