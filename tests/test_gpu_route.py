"""The routing kernel of the expert-parallel layer (peer_route_tuples) against the plain tensor form of
the same logic (llm720_b200/sharded.py: route_tuples_blocks), which the gloo CPU test checks against the
variable-length routing and the oracle; the expert stage reading received blocks in place
(peer_gather_eval_routed) against the list form (peer_gather_eval_partial); and the query+selection stage
entry that feeds them (peer_select_tokens) against the whole layer's selection.  Integer work: bit-exact."""
import pytest
import torch

from llm720_b200 import PeerOp, sharded, synthetic as syn
from _util import make_op, op_weights

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("T,E,world,rows", [(8, 256, 8, 524288), (5, 6, 4, 8), (64, 256, 2, 2097152), (40, 48, 3, 100),
                                             (1, 1, 1, 7), (3, 33, 2, 50)])
def test_route_kernel_equals_the_tensor_form(cuda_device, T, E, world, rows):
    g = torch.Generator().manual_seed(T * 1000 + E)
    ids = torch.randint(0, world * rows, (T, E), generator=g)
    if T > 2:
        ids[2] = rows // 2                                  # one token sends everything to rank 0, duplicates included
    w = torch.rand(T, E, generator=g)
    ids_d, w_d = ids.to(torch.int32).to(cuda_device), w.to(cuda_device)
    want = sharded.route_tuples_blocks(ids_d, w_d, rows, world)
    got = sharded.route_tuples_native(ids_d, w_d, rows, world)
    torch.cuda.synchronize()
    assert got.shape == (world, sharded.block_words(T, E))
    assert torch.equal(got, want)                          # same slot order, same zero padding, same counts
    assert int(got[:, 2 * T * E:].sum()) == T * E          # every tuple went to exactly one owner


def test_route_drops_ids_outside_the_table(cuda_device):
    ids = torch.tensor([[0, 5, -1, 16, 3]], dtype=torch.int32, device=cuda_device)
    w = torch.ones(1, 5, device=cuda_device)
    send = sharded.route_tuples_native(ids, w, 8, 2)          # table of 16 rows on 2 ranks
    assert send[:, 10:].flatten().tolist() == [3, 0]
    assert send[0, :3].tolist() == [0, 5, 3]


@pytest.mark.parametrize("T,world", [(8, 8), (32, 2), (50, 4)])
def test_routed_evaluation_equals_the_list_form(cuda_device, T, world):
    """peer_gather_eval_routed reads the received blocks in place; peer_gather_eval_partial takes the same lists
    as plain arrays.  Same kernel, same order of additions: bit-identical partial sums, in the split-token
    form (few tokens) and the warp-per-token form."""
    torch.manual_seed(T)
    D, H, k, rows = 1024, 4, 8, 512
    E = H * k
    op = PeerOp(input_dim=D, output_dim=D, num_heads=H, query_dim=32, product_key_dim=(64, 64), top_k=k,
                act_dtype=torch.bfloat16, table_dtype=torch.bfloat16, max_tokens=T * world, device=cuda_device)
    U = (torch.randn(rows, D) * D ** -0.5).bfloat16().to(cuda_device)
    V = (torch.randn(rows, D) * D ** -0.5).bfloat16().to(cuda_device)
    x = torch.randn(T * world, D).bfloat16().to(cuda_device)
    # what `world` peers would send this rank: each owns T tokens and this rank owns rows [0, rows) of world*rows
    blocks = []
    for b in range(world):
        ids = torch.randint(0, world * rows, (T, E))
        blocks.append(sharded.route_tuples_blocks(ids, torch.rand(T, E), rows, world)[0])
    recv = torch.stack(blocks).to(cuda_device).contiguous()
    got = op.gather_eval_routed(x, recv, world, T, U, V)
    l_ids, l_w, l_cnt = sharded.lists_from_blocks(recv, T, E)
    want = op.gather_eval_partial(x, l_ids, l_w.contiguous(), l_cnt, U, V)
    op.query_status()
    assert torch.equal(got, want)
    ref = torch.zeros(T * world, D)
    ic, wc, cc, xc, Uc, Vc = l_ids.cpu(), l_w.cpu(), l_cnt.cpu(), x.cpu().float(), U.cpu().float(), V.cpu().float()
    for t in range(0, T * world, 7):
        for j in range(int(cc[t])):
            r = int(ic[t, j])
            ref[t] += wc[t, j] * torch.nn.functional.gelu(Uc[r] @ xc[t]) * Vc[r]
        assert torch.allclose(got[t].cpu(), ref[t], rtol=1e-4, atol=1e-5)


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
    ids2 = torch.empty_like(ids)
    sc2 = torch.empty_like(sc)
    t = op._tensors(x, w, None, ids2, sc2)
    import ctypes as C
    HK = cfg.num_heads * cfg.top_k
    ids32 = torch.empty(cfg.tokens, HK, dtype=torch.int32, device=cuda_device)
    wts = torch.empty(cfg.tokens, HK, dtype=torch.float32, device=cuda_device)
    rc = op.lib.peer_select_tokens(op.handle, C.byref(t), cfg.tokens, C.c_void_p(ids32.data_ptr()), C.c_void_p(wts.data_ptr()),
                                   C.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0
    op.query_status()
    # the stage entry runs the query and selection kernels of the whole layer: same lists (compared with the
    # near-tie rule all the same, so that the test states the contract and not the implementation)
    from oracle import peer_oracle as orc
    rows, exact, near, bad = orc.compare_selection(ids2.cpu(), ids.cpu(), sc.cpu(), sc2.cpu())
    assert bad == 0 and exact >= 0.99 * rows, (rows, exact, near, bad)
    assert torch.allclose(sc2, sc, rtol=0, atol=2e-6)
    assert torch.equal(ids32.view(ids.shape).long(), ids2)                      # int32 and int64 outputs agree
    assert torch.allclose(wts.view(sc.shape), torch.softmax(sc2, -1), rtol=1e-6, atol=1e-7)
    ids32b, wtsb = op.select_tokens(x, w)                                        # the wrapper, and determinism
    assert torch.equal(ids32b, ids32) and torch.equal(wtsb, wts)
