"""Host logic of the expert-parallel layer (tuple routing, all-to-all, per-token packing,
reduce-scatter) with two CPU ranks over gloo.  The per-rank kernels are replaced by oracle
arithmetic here (test scaffolding only); the GPU version of this test is
tests/multi_gpu_check.py, run under torchrun on two GPUs."""
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from llm720_b200 import sharded, synthetic as syn
from oracle import peer_oracle as orc
from _util import oracle_shape, oracle_weights


def _cpu_layer():
    cfg = syn.PeerConfig("sh", 64, 96, 4, 32, (16, 16), 8, torch.float32, torch.float32, 1, 12)
    return cfg, syn.make_weights(cfg, 21, "cpu", random_affine=True), syn.make_input(cfg, 21, "cpu")


def _rank_main(rank, world, port, result_q, static_shapes=True):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.set_num_threads(2)
        cfg, sd, x = _cpu_layer()
        shape, w = oracle_shape(cfg), oracle_weights(sd)
        rows = cfg.num_experts // world
        U = sd["expert_down.weight"][rank * rows:(rank + 1) * rows]
        V = sd["expert_up.weight"][rank * rows:(rank + 1) * rows]
        t_local = cfg.tokens // world
        x_local = x.view(cfg.tokens, -1)[rank * t_local:(rank + 1) * t_local]

        def select_fn(xl):
            q = orc.make_queries(xl.unsqueeze(0), w, shape)
            ids, raw = orc.select(q, w.sub_keys, cfg.top_k, cfg.product_key_dim, index_mode="product")
            return ids.view(xl.shape[0], -1), torch.softmax(raw, -1).view(xl.shape[0], -1)

        def eval_fn(x_all, ids, wt, cnt):
            out = torch.zeros(x_all.shape[0], cfg.output_dim)
            for t in range(x_all.shape[0]):
                for j in range(int(cnt[t])):
                    r = int(ids[t, j])
                    assert 0 <= r < rows
                    out[t] += wt[t, j] * torch.nn.functional.gelu(U[r] @ x_all[t]) * V[r]
            return out

        out = sharded.sharded_forward(x_local, select_fn, eval_fn, cfg.num_experts, static_shapes=static_shapes)
        ref, _, _ = orc.forward(x, w, shape, "product")
        ref = ref.view(cfg.tokens, -1)[rank * t_local:(rank + 1) * t_local]
        result_q.put((rank, float((out - ref).abs().max()), float(ref.abs().max())))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("static_shapes", [True, False])
def test_two_cpu_ranks_equal_single_device(static_shapes):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + os.getpid() % 2000 + int(static_shapes)
    procs = [ctx.Process(target=_rank_main, args=(r, 2, port, q, static_shapes)) for r in range(2)]
    [p.start() for p in procs]
    res = [q.get(timeout=180) for _ in procs]
    [p.join(60) for p in procs]
    assert all(p.exitcode == 0 for p in procs)
    for rank, err, mag in res:
        assert err <= 1e-5 * max(mag, 1.0), (rank, err, mag)


def test_route_and_pack_roundtrip():
    torch.manual_seed(0)
    T, HK, world, rows = 5, 6, 4, 8
    ids = torch.randint(0, world * rows, (T, HK))
    w = torch.rand(T, HK)
    send, counts = sharded.route_tuples(ids, w, token_offset=10, rows=rows, world=world)
    assert int(counts.sum()) == T * HK and send.shape == (T * HK, 3)
    owner = torch.repeat_interleave(torch.arange(world), counts)
    glob = owner * rows + send[:, 1]
    # every (token, id, weight) tuple survives routing exactly once
    got = sorted(zip((send[:, 0] - 10).tolist(), glob.tolist(), send[:, 2].contiguous().view(torch.float32).tolist()))
    want = sorted(zip(torch.arange(T).repeat_interleave(HK).tolist(), ids.reshape(-1).tolist(), w.reshape(-1).tolist()))
    assert got == want
    # packing what one owner would receive
    mine = send[owner == 2]
    mine[:, 0] -= 10
    p_ids, p_w, p_cnt = sharded.pack_received(mine, T)
    assert int(p_cnt.sum()) == mine.shape[0] and p_ids.shape == p_w.shape
    for t in range(T):
        exp = sorted((int(i) - 2 * rows, float(x)) for i, x in zip(ids[t], w[t]) if 2 * rows <= int(i) < 3 * rows)
        have = sorted((int(p_ids[t, j]), float(p_w[t, j])) for j in range(int(p_cnt[t])))
        assert exp == have
    e_ids, e_w, e_cnt = sharded.pack_received(torch.empty(0, 3, dtype=torch.int32), 3)
    assert e_ids.shape == (3, 1) and int(e_cnt.sum()) == 0


def test_block_routing_matches_the_variable_length_routing():
    """The fixed-shape blocks ([local row ids | weight bits | counts] per destination) carry exactly the tuples
    the variable-length routing sends, token by token and in slot order."""
    torch.manual_seed(1)
    T, E, world, rows = 6, 8, 4, 16
    ids = torch.randint(0, world * rows, (T, E))
    ids[2] = 5                                      # one token sends everything to one owner
    w = torch.rand(T, E)
    send = sharded.route_tuples_blocks(ids, w, rows, world)
    assert send.shape == (world, sharded.block_words(T, E)) and send.dtype == torch.int32
    dyn, counts = sharded.route_tuples(ids, w, 0, rows, world)
    owner_of = torch.repeat_interleave(torch.arange(world), counts)
    for owner in range(world):
        a_ids, a_w, a_cnt = sharded.lists_from_blocks(send[owner:owner + 1], T, E)
        mine = dyn[owner_of == owner]
        b_ids, b_w, b_cnt = sharded.pack_received(mine, T)
        assert torch.equal(a_cnt, b_cnt)
        for t in range(T):
            n = int(a_cnt[t])
            assert a_ids[t, :n].tolist() == b_ids[t, :n].tolist()          # same order: slot order
            assert a_w[t, :n].tolist() == b_w[t, :n].tolist()
            assert a_ids[t, n:].abs().sum() == 0 and a_w[t, n:].abs().sum() == 0
    # a received set of blocks is already the list of every token: block b, row t = global token b*T + t
    recv = torch.stack([send[1], send[1]])
    g_ids, g_w, g_cnt = sharded.lists_from_blocks(recv, T, E)
    assert g_ids.shape == (2 * T, E) and torch.equal(g_cnt[:T], g_cnt[T:])


def test_uneven_split_is_rejected():
    with pytest.raises(ValueError):
        sharded.rows_per_rank(10, 4)
