"""The two routing kernels of the expert-parallel layer (peer_route_tuples, peer_pack_tuples) against the
plain tensor form of the same logic (llm720_b200/sharded.py: route_tuples_static, pack_received_static),
which the gloo CPU test checks against the oracle, and the query+selection stage entry that feeds them
(peer_select_tokens) against the whole layer's selection.  Integer work: bit-exact."""
import pytest
import torch

from llm720_b200 import sharded, synthetic as syn
from _util import make_op, op_weights

pytestmark = pytest.mark.gpu


def _as_sets(ids, w, cnt):
    return [sorted(zip(ids[t, :int(cnt[t])].tolist(), w[t, :int(cnt[t])].tolist())) for t in range(ids.shape[0])]


@pytest.mark.parametrize("T,HK,world,rows", [(8, 256, 8, 524288), (5, 6, 4, 8), (64, 256, 2, 2097152), (40, 48, 3, 100),
                                              (1, 1, 1, 7)])
def test_route_and_pack_kernels_equal_the_tensor_form(cuda_device, T, HK, world, rows):
    g = torch.Generator().manual_seed(T * 1000 + HK)
    ids = torch.randint(0, world * rows, (T, HK), generator=g)
    if T > 2:
        ids[2] = rows // 2                                  # one token sends everything to rank 0, duplicates included
    w = torch.rand(T, HK, generator=g)
    dev = cuda_device
    ids_d, w_d = ids.to(torch.int32).to(dev), w.to(dev)
    want = sharded.route_tuples_static(ids_d, w_d, 11, rows, world)
    got = sharded.route_tuples_native(ids_d, w_d, 11, rows, world)
    torch.cuda.synchronize()
    assert got.shape == (world, T * HK, 3)
    assert torch.equal(got[..., 0], want[..., 0])          # same stable order, same padding
    used = got[..., 0] >= 0
    assert torch.equal(got[used], want[used])
    # receiving side: what arrives is [world, cap, 3] from the peers; reuse the buckets as if received
    recv = got.clone()
    recv[..., 0] = torch.where(recv[..., 0] >= 0, recv[..., 0] - 11, recv[..., 0])
    a = sharded.pack_received_native(recv, T, HK)
    b = sharded.pack_received_static(recv, T, HK)
    torch.cuda.synchronize()
    assert torch.equal(a[2], b[2])
    assert _as_sets(a[0].cpu(), a[1].cpu(), a[2].cpu()) == _as_sets(b[0].cpu(), b[1].cpu(), b[2].cpu())
    # every tuple arrives exactly once: global id = bucket * rows + local row
    owner = torch.arange(world, device=dev).view(world, 1).expand(world, T * HK)
    glob = (owner * rows + got[..., 1])[used]
    have = sorted(zip((got[..., 0][used] - 11).tolist(), glob.tolist(), got[..., 2][used].view(torch.float32).tolist()))
    exp = sorted(zip(torch.arange(T).repeat_interleave(HK).tolist(), ids.reshape(-1).tolist(), w.reshape(-1).tolist()))
    assert have == exp
    # a list shorter than the tuples of a token keeps the first ones and reports the capacity
    c = sharded.pack_received_native(recv, T, max(HK // 2, 1))
    assert int(c[2].max()) <= max(HK // 2, 1)


def test_route_drops_ids_outside_the_table(cuda_device):
    ids = torch.tensor([[0, 5, -1, 16, 3]], dtype=torch.int32, device=cuda_device)
    w = torch.ones(1, 5, device=cuda_device)
    send = sharded.route_tuples_native(ids, w, 0, 8, 2)        # table of 16 rows on 2 ranks
    assert int((send[..., 0] >= 0).sum()) == 3
    assert send[0, :3, 1].tolist() == [0, 5, 3]


def test_select_tokens_equals_the_layers_selection(cuda_device):
    cfg = syn.scaled(syn.CONFIGS["c4"], product_key_dim=(256, 128), batch=24, seq=1)
    sd = syn.make_weights(cfg, 61, cuda_device, random_affine=True)
    x = syn.make_input(cfg, 61, cuda_device).view(cfg.tokens, -1)
    op = make_op(cfg, cuda_device, "product")
    w = op_weights(sd, cuda_device)
    out = torch.empty(cfg.tokens, cfg.output_dim, dtype=cfg.dtype, device=cuda_device)
    ids = torch.empty(cfg.tokens, cfg.num_heads, cfg.top_k, dtype=torch.int64, device=cuda_device)
    sc = torch.empty(cfg.tokens, cfg.num_heads, cfg.top_k, dtype=torch.float32, device=cuda_device)
    op.forward(x, w, out, ids, sc)
    ids32, wts = op.select_tokens(x, w)
    op.query_status()
    assert torch.equal(ids32.view(ids.shape).long(), ids)
    assert torch.allclose(wts.view(sc.shape), torch.softmax(sc, -1), rtol=1e-6, atol=1e-7)
