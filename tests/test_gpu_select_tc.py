"""Adversarial inputs for the tensor-core selection kernel, through the C ABI stage entry
(peer_select on a bf16 handle runs the same kernels as the whole layer).

What is forced, and how the test knows it fired (peer_select_stats):
  * candidate lists longer than 32 entries that continue in the shared pool (blocks of identical
    high-scoring sub-keys);
  * rows that lose a candidate - a full pool (hundreds of identical keys) or one key that is a hit for
    more than 8 of the 32 rows a scan lane serves (a "popular" key) - and are redone by the exact
    CUDA-core kernel;
  * sub-key tables whose size is not a multiple of the 128-key chunk (the last TMA box runs off the
    table, keys past the end must lose every comparison);
  * k in {1, 4, 8, 16}, query_dim 128 and 256, row counts that are not a multiple of the 128-row tile.

Oracle: the reference's selection (experts.py:138-285 restated in oracle/peer_oracle.py) in fp32 on the
same bf16-representable keys.  Bounds: raw scores within 3e-6; ids equal as ordered lists except inside
groups of (nearly) tied scores; independent of ties, every returned id must own the score returned
with it (the id is decoded into its two sub-key indices and the two oracle sub-scores are added).
"""
import pytest
import torch

from llm720_b200 import synthetic as syn
from oracle import peer_oracle as orc
from _util import make_op

pytestmark = pytest.mark.gpu


WIDE_ROWS = 148 * 32 + 64      # batches of more (token, head) rows than this take tiles of 128 rows, smaller ones of 32


@pytest.fixture(params=["tiles_of_32_rows", "tiles_of_128_rows"])
def wide(request):
    return request.param == "tiles_of_128_rows"


def _run(dev, q, keys, k, mode="product", norm_keys=True, norm_query=True, wide=False):
    """q fp32 [T, H, Q], keys two bf16 tables -> (ids, scores, (pooled lists, refined rows), oracle ids, oracle scores).
    ``wide``: random filler tokens follow q, enough for the kernel to choose its 128-row tiles; only q's rows are
    returned and checked."""
    T, H, Q = q.shape
    n = (keys[0].shape[0], keys[1].shape[0])
    q_run = q
    if wide and T * H <= WIDE_ROWS:
        q_run = torch.cat([q, _queries((WIDE_ROWS + H) // H - T + 1, H, Q, 999)])
    cfg = syn.PeerConfig("seltc", 64, 64, H, Q, n, k, torch.bfloat16, torch.bfloat16, 1, q_run.shape[0])
    op = make_op(cfg, dev, mode, norm_keys=norm_keys, norm_query=norm_query)
    op.select_stats()
    ids, sc = op.select(q_run.to(dev).contiguous(), keys[0].to(dev), keys[1].to(dev))
    op.query_status()
    stats = op.select_stats()
    ids, sc = ids[:T], sc[:T]
    kf = [kt.float() for kt in keys]
    with torch.no_grad():
        o_ids, o_sc = orc.select(q.unsqueeze(0), kf, k, n, norm_keys, norm_query, mode)
        s0, s1 = orc.sub_key_scores(q.unsqueeze(0), kf, norm_keys, norm_query)
    o_ids, o_sc = o_ids.view(T, H, k), o_sc.view(T, H, k)
    ids_c, sc_c = ids.cpu(), sc.cpu()
    assert ids_c.shape == (T, H, k) and torch.isfinite(sc_c).all()
    tol = 3e-6 * max(1.0, float(o_sc.abs().max()))          # scores of unnormalised operands are not bounded by 2
    assert torch.allclose(sc_c, o_sc, rtol=0, atol=tol), float((sc_c - o_sc).abs().max())
    rows, exact, near, bad = orc.compare_selection(ids_c, o_ids, o_sc, sc_c)
    assert bad == 0, (rows, exact, near, bad)
    if mode == "product":       # every id owns its score, whatever order ties came out in
        i0, i1 = ids_c // n[1], ids_c % n[1]
        assert int(i0.max()) < n[0] and int(ids_c.min()) >= 0
        own = torch.gather(s0.view(T, H, -1), 2, i0) + torch.gather(s1.view(T, H, -1), 2, i1)
        assert torch.allclose(own, sc_c, rtol=0, atol=tol), float((own - sc_c).abs().max())
        # no (i0, i1) pair is returned twice
        flat = ids_c.view(-1, k).sort(-1).values
        assert bool((flat[:, 1:] != flat[:, :-1]).all())
    return ids_c, sc_c, stats, exact, rows


def _keys(n, w, seed):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(n, w, generator=g) * w ** -0.5).bfloat16()


def _queries(T, H, Q, seed):
    return torch.randn(T, H, Q, generator=torch.Generator().manual_seed(seed))


@pytest.mark.parametrize("n_keys,k,H,Q,T", [((1024, 1024), 16, 8, 256, 77), ((1000, 130), 16, 3, 256, 50),
                                             ((129, 1024), 8, 2, 128, 67), ((128, 128), 1, 1, 128, 5),
                                             ((256, 384), 4, 5, 128, 33), ((640, 512), 8, 4, 256, 129)])
@pytest.mark.parametrize("mode", ["reference", "product"])
def test_ragged_grids_small_k_and_partial_tiles(cuda_device, n_keys, k, H, Q, T, mode, wide):
    keys = [_keys(n_keys[0], Q // 2, 1), _keys(n_keys[1], Q // 2, 2)]
    q = _queries(T, H, Q, 3 + k)
    _, _, stats, exact, rows = _run(cuda_device, q, keys, k, mode, wide=wide)
    assert exact >= 0.99 * rows


@pytest.mark.parametrize("norm_keys,norm_query", [(True, False), (False, True), (False, False)])
def test_normalisation_switches_on_the_tensor_core_path(cuda_device, norm_keys, norm_query, wide):
    """norm_keys / norm_query off (experts.py:153-163): without unit queries the first pass has no error bound for
    a dropped term and contracts all three; without key normalisation the scale factors are 1."""
    n_keys, k, H, Q, T = (1024, 640), 16, 4, 256, 70
    keys = [_keys(n_keys[0], Q // 2, 5), _keys(n_keys[1], Q // 2, 6)]
    q = _queries(T, H, Q, 7)
    _, _, _, exact, rows = _run(cuda_device, q, keys, k, "product", norm_keys, norm_query, wide=wide)
    assert exact >= 0.99 * rows


def test_identical_keys_overflow_the_list_into_the_pool(cuda_device, wide):
    """40 copies of one sub-key, spread over the table: in the rows whose query points at that key all 40
    tie for first place, so the row's candidate list (32 slots) spills into the pool."""
    T, H, Q, n, k = 96, 2, 256, 1024, 16
    keys = [_keys(n, Q // 2, 11), _keys(n, Q // 2, 12)]
    dup = torch.arange(40) * 25 + 3                              # 40 rows of table 0, many key groups
    keys[0][dup] = keys[0][3].clone()
    q = _queries(T, H, Q, 13)
    hot = torch.arange(0, T, 9)                                   # a few rows per tile: the pool (64 entries) suffices
    q[hot, :, :Q // 2] = q[hot, :, :Q // 2] * 0.3 + 4.0 * keys[0][3].float()
    ids, sc, (pooled, refined), _, _ = _run(cuda_device, q, keys, k, wide=wide)
    assert pooled > 0, "the pool path did not fire"
    # the hot rows' best 16 all carry a copy of the duplicated key in dimension 0
    i0 = ids[hot] // n
    assert bool(torch.isin(i0, dup).all())


def test_hundreds_of_identical_keys_fill_the_pool_and_rows_are_redone_exactly(cuda_device, wide):
    T, H, Q, n, k = 40, 4, 256, 1024, 16
    keys = [_keys(n, Q // 2, 21), _keys(n, Q // 2, 22)]
    dup = torch.arange(300) * 3 + 1
    keys[1][dup] = keys[1][1].clone()
    q = _queries(T, H, Q, 23)
    q[:, :, Q // 2:] = q[:, :, Q // 2:] * 0.3 + 4.0 * keys[1][1].float()      # every row ties 300 ways
    ids, sc, (pooled, refined), _, _ = _run(cuda_device, q, keys, k, wide=wide)
    assert refined > 0, "no row went to the exact kernel"
    assert bool(torch.isin(ids % n, dup).all())


def test_a_popular_key_exceeds_one_lanes_staging_slots(cuda_device, wide):
    """One key that scores in the top 16 of every row: the scan lane that owns it has a hit in all 32 of
    its rows in one chunk, more than its 8 staging slots, so those rows go to the exact kernel."""
    T, H, Q, n, k = 64, 2, 128, 512, 8
    keys = [_keys(n, Q // 2, 31), _keys(n, Q // 2, 32)]
    q = _queries(T, H, Q, 33)
    q[:, :, :Q // 2] += 6.0 * keys[0][77].float()            # cosine with key 77 around 0.6 in every row
    ids, sc, (pooled, refined), _, _ = _run(cuda_device, q, keys, k, wide=wide)
    assert refined > 0, "the staging-slot overflow did not fire"
    assert float(((ids // n) == 77).any(-1).float().mean()) > 0.9


def test_clustered_scores_without_exact_ties(cuda_device, wide):
    """Keys drawn around a few centres (what trained sub-keys look like, unlike N(0, 1/d) noise): many
    scores sit just under each row's bound."""
    T, H, Q, n, k = 130, 4, 256, 1024, 16
    g = torch.Generator().manual_seed(41)
    centres = torch.randn(8, Q // 2, generator=g)
    keys = []
    for t in range(2):
        which = torch.randint(0, 8, (n,), generator=g)
        keys.append((centres[which] + 0.05 * torch.randn(n, Q // 2, generator=g)).bfloat16())
    q = _queries(T, H, Q, 43)
    _, _, (pooled, refined), exact, rows = _run(cuda_device, q, keys, k, wide=wide)
    assert pooled + refined > 0


def test_both_tile_shapes_give_the_same_lists(cuda_device):
    """A row's result does not depend on the rows it shares a tile with: the same queries alone (tiles of 32
    rows) and followed by filler tokens (tiles of 128 rows), bit for bit, tied rows included."""
    T, H, Q, n, k = 90, 4, 256, (1024, 640), 16
    keys = [_keys(n[0], Q // 2, 61), _keys(n[1], Q // 2, 62)]
    keys[0][torch.arange(20) * 40 + 7] = keys[0][7].clone()       # some exact ties
    q = _queries(T, H, Q, 63)
    q[::5, :, :Q // 2] = q[::5, :, :Q // 2] * 0.3 + 4.0 * keys[0][7].float()
    ids_a, sc_a, _, _, _ = _run(cuda_device, q, keys, k, wide=False)
    ids_b, sc_b, _, _, _ = _run(cuda_device, q, keys, k, wide=True)
    assert torch.equal(ids_a, ids_b) and torch.equal(sc_a, sc_b)


def test_stage_entry_equals_whole_layer_selection(cuda_device):
    """peer_select on a bf16 handle and peer_forward select with the same kernels: same ids and scores
    from the queries the layer itself projects."""
    cfg = syn.scaled(syn.CONFIGS["c2"], product_key_dim=(256, 384), batch=1, seq=150)
    from _util import op_weights
    sd = syn.make_weights(cfg, 51, cuda_device, random_affine=True)
    x = syn.make_input(cfg, 51, cuda_device).view(cfg.tokens, -1)
    op = make_op(cfg, cuda_device, "product")
    w = op_weights(sd, cuda_device)
    out = torch.empty(cfg.tokens, cfg.output_dim, dtype=cfg.dtype, device=cuda_device)
    ids = torch.empty(cfg.tokens, cfg.num_heads, cfg.top_k, dtype=torch.int64, device=cuda_device)
    sc = torch.empty(cfg.tokens, cfg.num_heads, cfg.top_k, dtype=torch.float32, device=cuda_device)
    op.forward(x, w, out, ids, sc)
    q = op.project_queries(x, w)
    ids2, sc2 = op.select(q, w["keys0"], w["keys1"])
    op.query_status()
    # (the two paths sum the squares of a query half in different orders: the last bit of a score may differ)
    rows, exact, near, bad = orc.compare_selection(ids2.cpu(), ids.cpu(), sc.cpu(), sc2.cpu())
    assert bad == 0 and exact >= 0.99 * rows, (rows, exact, near, bad)
    assert torch.allclose(sc, sc2, rtol=0, atol=2e-6)


def test_frozen_keys_are_prepared_once_and_anew_for_other_tables(cuda_device):
    """peer_freeze_keys: the key tables' derived data is reused for the same two tensors, recomputed for other
    tensors and after the flag is set again; results equal those of a handle that prepares them in every call."""
    T, H, Q, n, k = 48, 4, 256, (512, 384), 16
    keys = [_keys(n[0], Q // 2, 71).to(cuda_device), _keys(n[1], Q // 2, 72).to(cuda_device)]
    other = _keys(n[0], Q // 2, 73).to(cuda_device)
    q = _queries(T, H, Q, 74).to(cuda_device).contiguous()
    cfg = syn.PeerConfig("frozen", 64, 64, H, Q, n, k, torch.bfloat16, torch.bfloat16, 1, T)
    plain, frozen = make_op(cfg, cuda_device, "product"), make_op(cfg, cuda_device, "product")
    frozen.freeze_keys(True)
    want = plain.select(q, keys[0], keys[1])
    for _ in range(3):                                   # the first call prepares, the others reuse
        got = frozen.select(q, keys[0], keys[1])
        assert torch.equal(got[0], want[0]) and torch.equal(got[1], want[1])
    want_other = plain.select(q, other, keys[1])
    got = frozen.select(q, other, keys[1])               # another tensor: prepared anew
    assert torch.equal(got[0], want_other[0]) and torch.equal(got[1], want_other[1])
    assert not torch.equal(want_other[0], want[0])
    keys[0].copy_(other)                                 # in place: the caller's promise is broken ...
    frozen.select(q, keys[0], keys[1])
    frozen.freeze_keys(True)                             # ... and renewed: prepared anew
    got = frozen.select(q, keys[0], keys[1])
    assert torch.equal(got[0], want_other[0]) and torch.equal(got[1], want_other[1])
    frozen.query_status()

