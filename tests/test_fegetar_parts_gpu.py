"""Fegetar's mechanisms one by one on the GPU, each against the plain implementation (or a few
float64 lines in the test), with inputs made so that a fault shows: a far key that one score
singles out, keys on both sides of a page's edge and of a window's edge, the key just behind a
query, the first tokens, state that crosses a portion's edge and slots that are used again."""

import math

import pytest
import torch

from tests.fegetar_configs import FEG, fegetar_weights
from tests.plain import fegetar_plain as plain

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]
TOL = {torch.float32: 2e-5, torch.bfloat16: 2e-2}


def _dev(x, dtype=None):
    return x.to("cuda", dtype) if dtype is not None else x.to("cuda")


def _i32(values):
    return torch.tensor(list(values), dtype=torch.int32, device="cuda")


def _rel(got, want):
    return float((got.double().cpu() - want.double().cpu()).abs().max() / want.double().abs().max().clamp_min(1e-30))


# ---------------------------------------------------------------------------
# embedding: the pair table and the token kept between portions


def test_pair_hash_embedding_over_portions_and_reused_slots():
    from tokensprint_b200 import ops

    V, W, buckets, mp, mc = 50, 24, 13, 7, 3
    g = torch.Generator().manual_seed(0)
    embed, table = torch.randn(V, W, generator=g), torch.randn(buckets + 1, W, generator=g)
    weights = {"embed": embed, "bigram": table}
    cfg = {"embedding": {"bigram": {"buckets": buckets, "mul_prev": mp, "mul_cur": mc}}}
    seqs = {0: torch.randint(0, V, (11,), generator=g).tolist(), 1: torch.randint(0, V, (7,), generator=g).tolist(),
            2: torch.randint(0, V, (5,), generator=g).tolist()}
    want = {k: plain.embed(v, weights, cfg) for k, v in seqs.items()}
    last = torch.full((2,), 77, dtype=torch.int32, device="cuda")  # two slots; stale content must not matter
    # steps: (sequence, first, count, slot); sequence 2 takes over slot 0 after sequence 0 has ended
    steps = [[(0, 0, 4, 0), (1, 0, 1, 1)], [(1, 1, 2, 1), (0, 4, 1, 0)], [(0, 5, 6, 0), (1, 3, 4, 1)], [(2, 0, 2, 0)], [(2, 2, 3, 0)]]
    for step in steps:
        ids, pos, sidx, cu, slots = [], [], [], [0], []
        for b, (s, first, count, slot) in enumerate(step):
            ids += seqs[s][first : first + count]
            pos += list(range(first, first + count))
            sidx += [b] * count
            cu.append(len(ids))
            slots.append(slot)
        ids_d = _i32(ids)
        hidden = torch.empty((len(ids), W), device="cuda", dtype=torch.float32)
        ops.embed_gather(hidden, _dev(embed), ids_d)
        ops.pair_hash_embed(hidden, _dev(table), ids_d, _i32(pos), _i32(sidx), _i32(cu), _i32(slots), last, buckets, mp, mc, V)
        row = 0
        for s, first, count, _ in step:
            assert torch.allclose(hidden[row : row + count].cpu().double(), want[s][first : first + count], atol=1e-6), (s, first)
            row += count


def test_pair_hash_embedding_takes_large_multipliers():
    from tokensprint_b200 import ops

    V, W, buckets, mp, mc = 200000, 8, 99991, 2147483629, 2147483587
    table = torch.arange(buckets + 1, dtype=torch.float32)[:, None].repeat(1, W)
    ids = [199999, 123456, 7]
    hidden = torch.zeros((3, W), device="cuda")
    ops.pair_hash_embed(hidden, _dev(table), _i32(ids), _i32([0, 1, 2]), _i32([0, 0, 0]), _i32([0, 3]), _i32([0]),
                        torch.zeros(1, dtype=torch.int32, device="cuda"), buckets, mp, mc, V)
    assert hidden[:, 0].tolist() == [float(r) for r in plain.pair_rows(ids, mp, mc, buckets)]


# ---------------------------------------------------------------------------
# norms and small element-wise kernels


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width", [70, 72, 256, 1000, 4100])
def test_norm_on_the_branch(dtype, width):
    from tokensprint_b200 import ops

    g = torch.Generator().manual_seed(width)
    hidden, branch, w = torch.randn(5, width, generator=g), torch.randn(5, width, generator=g) * 3, torch.randn(width, generator=g) * 0.1
    branch = branch.to(dtype)
    want = hidden.double() + plain.norm_around_zero(branch.double(), w.double(), 1e-5)
    h, rounded = _dev(hidden.clone()), torch.empty((5, width), device="cuda", dtype=dtype)
    ops.rmsnorm_add(_dev(branch), _dev(1.0 + w), h, 1e-5, rounded)
    assert _rel(h, want) < 1e-6
    assert torch.equal(rounded, h.to(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
def test_activations(dtype):
    from tokensprint_b200 import ops

    g = torch.Generator().manual_seed(3)
    x = (torch.randn(7, 50, generator=g) * 3).to(dtype)
    out = torch.empty_like(x, device="cuda")
    ops.gelu_tanh(_dev(x), out)
    assert _rel(out, plain.gelu_tanh(x.double())) < TOL[dtype]
    gu = (torch.randn(7, 2 * 30, generator=g) * 3).to(dtype)
    act = torch.empty((7, 30), device="cuda", dtype=dtype)
    ops.capped_glu(_dev(gu), act, 1.5, 1.702)
    a, b = gu[:, :30].double().clamp(max=1.5), gu[:, 30:].double().clamp(-1.5, 1.5)
    assert _rel(act, a * torch.sigmoid(1.702 * a) * (b + 1)) < TOL[dtype]
    table, ids = torch.randn(9, 40, generator=g).to(dtype), [8, 0, 3, 3, 5, 1, 2]
    y = _dev(x[:, :12].contiguous())
    ops.gelu_gate_rows(y, _dev(table), _i32(ids), 24)
    assert _rel(y, plain.gelu_tanh(x[:, :12].double()) * table[ids][:, 24:36].double()) < TOL[dtype]


# ---------------------------------------------------------------------------
# latent attention: the kernels on made-up rows


def _paged(rows: torch.Tensor, page: int, dtype, seed: int, spare: int = 3):
    """Puts a sequence's cache rows [N, D] into pages in a shuffled order; returns pool and table."""
    N, D = rows.shape
    n_pages = -(-N // page)
    g = torch.Generator().manual_seed(seed)
    order = torch.randperm(n_pages + spare, generator=g)[:n_pages]
    pool = torch.full(((n_pages + spare), page, D), float("nan"), dtype=dtype)
    for j in range(N):
        pool[order[j // page], j % page] = rows[j].to(dtype)
    return pool, order.tolist()


def _attention_reference(q, rows, positions, rank, scale, window, gates):
    out = torch.zeros(q.shape[0], q.shape[1], rank, dtype=torch.float64)
    for t, p in enumerate(positions):
        lo = max(0, p - window + 1) if window else 0
        K = rows[lo : p + 1].double()
        w = torch.softmax(q[t].double() @ K.T * scale, -1)
        out[t] = (w @ K[:, :rank]) * gates[t].double()[:, None]
    return out


ATTENTION_CASES = [
    # rank, rot, heads, page, context, queries (the step's tokens are the last `queries` positions), window
    (40, 16, 3, 16, 700, 1, 0),
    (40, 16, 3, 16, 700, 5, 0),
    (18, 6, 1, 8, 130, 33, 0),
    (32, 16, 8, 16, 257, 64, 0),
    (64, 32, 4, 16, 300, 2, 0),
    (40, 16, 3, 16, 200, 7, 37),
    (26, 10, 5, 32, 96, 96, 0),
    (48, 16, 6, 16, 333, 40, 0),
    (128, 32, 16, 32, 520, 3, 0),
    (64, 16, 2, 64, 400, 1, 100),
    (512, 64, 4, 16, 200, 9, 0),
]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rank, rot, H, page, N, Q, window", ATTENTION_CASES)
def test_latent_attention_finds_the_one_key(dtype, rank, rot, H, page, N, Q, window):
    """All rows are small noise except one whose score stands out for one (query, head): the output
    there must be that row's latent.  The one key sits far away, on both sides of page edges, among
    the first tokens, at the query's own place, just behind the query (not to be seen), and on
    both sides of the window's edge."""
    from tokensprint_b200 import ops

    D = rank + rot
    g = torch.Generator().manual_seed(N + Q)
    first = N - Q
    positions = list(range(first, N))
    special = sorted({0, 1, page - 1, page, page + 1, 2 * page - 1, N // 2, first - 1, first, N - 2, N - 1} & set(range(N)))
    if window:
        special = sorted(set(special) | {max(0, N - 1 - window), max(0, N - window), max(0, N - window + 1)})
    for j_star in special:
        rows = torch.randn(N, D, generator=g) * 0.05
        u = torch.randn(D, generator=g)
        u = u / u.norm()
        rows[j_star] = 6.0 * u + rows[j_star] * 0.1
        rows[j_star, :rank] += torch.linspace(-1, 1, rank)  # a latent that is easy to tell from noise
        q = torch.randn(Q, H, D, generator=g) * 0.05
        t_star, a_star = Q - 1, H - 1
        q[t_star, a_star] = 6.0 * u
        if Q > 1 and first <= j_star < N - 1:
            q[j_star - first, 0] = 6.0 * u  # the query at the key's own place sees it; the one before must not
            if j_star - first >= 1:
                q[j_star - first - 1, 0] = 6.0 * u
        gates = torch.rand(Q, H, generator=g) * 0.5 + 0.5
        q, rows = q.to(dtype).float(), rows.to(dtype).float()
        want = _attention_reference(q, rows, positions, rank, 1.0, window, gates)
        pool, table = _paged(rows, page, dtype, j_star)
        out = torch.empty((Q, H, rank), device="cuda", dtype=dtype)
        ops.latent_attention_simple(_dev(q, dtype), _dev(pool), out, _dev(gates), _i32(positions), _i32([0] * Q), _i32(table).view(1, -1),
                                    page, H, rank, rot, 1.0, window)
        err = _rel(out, want)
        assert err < TOL[dtype], f"key {j_star} of {N} (page {page}, window {window}): error {err:.3g}"
        if dtype == torch.bfloat16 and ops.latent_attention_mma_supported(rank, rot):
            # the tensor-core kernel: the same rows as a second sequence of a batch whose first sequence is
            # short, whole and cut into key ranges
            short = 5
            q2 = torch.cat([q[:1].expand(short, H, D), q]).contiguous()
            g2 = torch.cat([gates[:1].expand(short, H), gates]).contiguous()
            tables = torch.full((2, len(table)), -1, dtype=torch.int32)
            tables[0, 0] = table[0]
            tables[1] = torch.tensor(table, dtype=torch.int32)
            for splits in (1, 3, 8):
                if splits > 1 and Q > 4:
                    continue
                out2 = torch.full((short + Q, H, rank), float("nan"), device="cuda", dtype=dtype)
                ops.latent_attention_mma(_dev(q2, dtype), _dev(pool), out2, _dev(g2), _i32([0, short, short + Q]), _i32([short, N]),
                                         _dev(tables), page, 2, max(short, Q), H, rank, rot, 1.0, window, splits)
                err = _rel(out2[short:], want)
                assert err < TOL[dtype], f"tensor cores, {splits} splits, key {j_star} of {N} (page {page}, window {window}): error {err:.3g}"
                assert bool(torch.isfinite(out2[:short].float()).all())


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("tag, layer", [("a", 0), ("b", 0), ("b", 1), ("c", 1)])
def test_latent_mixer_whole_prompt(dtype, tag, layer):
    """The mixer part alone (projection, prepare kernel, absorbing products, attention, value
    products, output) against the plain function that rebuilds keys and values per head."""
    from tokensprint_b200.models.fegetar import build_fegetar_spec, FegetarConfig
    from tokensprint_b200.parts.base import BuildContext, GroupTables, LayerCache, StepContext, build_part

    cfg = FEG[tag]
    W = fegetar_weights(cfg, 17, sharp=2.0)
    spec = build_fegetar_spec(FegetarConfig.from_dict(cfg)).layers[layer].params["mixer"]
    mixer = build_part("mixer", spec, BuildContext(torch.device("cuda"), dtype))
    mixer.load({s.name: _dev(W[s.name], torch.float32 if s.role == "vector" else dtype) for s in mixer.tensor_specs()})
    T, page = 45, 16
    x = torch.randn(T, cfg["width"], generator=torch.Generator().manual_seed(5)).to(dtype)
    want = plain.latent_attention(x.double(), list(range(T)), {k: v.double() for k, v in W.items()}, f"l{layer}.mix.", cfg["layers"][layer]["mixer"],
                                  cfg["norm"]["eps"])
    pages = [2, 0, 3]
    pool = torch.full((4, page, mixer.key_dim), float("nan"), device="cuda", dtype=dtype)
    slots = [pages[j // page] * page + j % page for j in range(T)]
    step = StepContext(num_tokens=T, num_seqs=1, token_ids=_i32([0] * T), positions=_i32(range(T)), seq_index=_i32([0] * T),
                       cu_seqlens_q=_i32([0, T]), context_lens=_i32([T]), state_slots=_i32([0]),
                       groups=[GroupTables(_i32(pages).view(1, -1), _i32(slots))], page_size=page, max_seqlen_q=T, max_context_len=T)
    got = mixer.forward(_dev(x), step, LayerCache(group=0, k_pages=pool, writes=True))
    assert _rel(got, want) < (2e-5 if dtype == torch.float32 else 3e-2)


# ---------------------------------------------------------------------------
# routed experts


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("tag, layer, tokens", [("a", 0, 1), ("a", 0, 70), ("b", 1, 9), ("c", 0, 200), ("c", 1, 3)])
def test_routed_experts(dtype, tag, layer, tokens):
    from tokensprint_b200.models.fegetar import build_fegetar_spec, FegetarConfig
    from tokensprint_b200.parts.base import BuildContext, build_part

    cfg = FEG[tag]
    W = fegetar_weights(cfg, 23)
    spec = build_fegetar_spec(FegetarConfig.from_dict(cfg)).layers[layer].params["feed_forward"]
    part = build_part("feed_forward", spec, BuildContext(torch.device("cuda"), dtype))
    part.load({s.name: _dev(W[s.name], torch.float32 if s.role == "vector" else dtype) for s in part.tensor_specs()})
    x32 = torch.randn(tokens, cfg["width"], generator=torch.Generator().manual_seed(tokens))
    x = x32.to(dtype)
    want = plain.routed_ff(x.double(), {k: v.double() for k, v in W.items()}, f"l{layer}.mlp.", cfg["layers"][layer]["mlp"])
    got = part.forward(_dev(x), None, residual=_dev(x.float()))
    assert _rel(got, want) < (2e-5 if dtype == torch.float32 else 3e-2)
    # a token's result does not depend on the tokens beside it
    if tokens > 2:
        alone = part.forward(_dev(x[1:2]), None, residual=_dev(x[1:2].float()))
        assert _rel(alone, got[1:2]) < 1e-6 if dtype == torch.float32 else torch.equal(alone, got[1:2])


def test_router_picks_by_score_and_breaks_ties_by_index():
    from tokensprint_b200 import ops

    logits = torch.tensor([[0.0, 2.0, -1.0, 2.0, 1.0], [5.0, -5.0, 0.5, 0.25, 0.125]], device="cuda")
    ids = torch.empty((2, 3), dtype=torch.int32, device="cuda")
    w = torch.empty((2, 3), dtype=torch.float32, device="cuda")
    ops.router_topk(logits, 3, False, ids, w)
    assert ids.tolist() == [[1, 3, 4], [0, 2, 3]]
    assert torch.allclose(w.cpu(), torch.sigmoid(torch.tensor([[2.0, 2.0, 1.0], [5.0, 0.5, 0.25]])))
    ops.router_topk(logits, 3, True, ids, w)
    assert torch.allclose(w.sum(-1).cpu(), torch.ones(2))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T, W, E, top", [(1, 72, 7, 3), (9, 256, 12, 1), (130, 1000, 33, 4), (5, 70, 4, 4), (600, 128, 9, 2), (2100, 64, 5, 1)])
def test_router_in_one_kernel(dtype, T, W, E, top):
    from tokensprint_b200 import ops

    g = torch.Generator().manual_seed(T)
    x, r = torch.randn(T, W, generator=g).to(dtype), torch.randn(E, W, generator=g) / W ** 0.5
    ids = torch.empty((T, top), dtype=torch.int32, device="cuda")
    w = torch.empty((T, top), dtype=torch.float32, device="cuda")
    ops.router(_dev(x), _dev(r), top, False, ids, w)
    score = torch.sigmoid(x.double() @ r.double().T)
    want_w, want_e = torch.topk(score, top, dim=-1)
    assert torch.equal(ids.cpu().long(), want_e)
    assert torch.allclose(w.cpu().double(), want_w, atol=1e-6)


@pytest.mark.parametrize("P, E, K, I", [(1, 3, 64, 48), (70, 5, 96, 200), (300, 4, 520, 72), (40, 9, 128, 24), (36, 3, 72, 136)])
def test_expert_products_on_tensor_cores_against_cuda_cores(P, E, K, I, monkeypatch):
    """The same plan through both kernels; bfloat16, float32 sums in both."""
    from tokensprint_b200 import ops

    g = torch.Generator().manual_seed(P)
    top = 2 if P % 2 == 0 else 1
    T = P // top
    x = torch.randn(T, K, generator=g).to(torch.bfloat16).cuda()
    gate, up = (torch.randn(E, I, K, generator=g) / K ** 0.5).to(torch.bfloat16).cuda(), (torch.randn(E, I, K, generator=g) / K ** 0.5).to(torch.bfloat16).cuda()
    down = (torch.randn(E, K, I, generator=g) / I ** 0.5).to(torch.bfloat16).cuda()
    ids = torch.stack([torch.randperm(E, generator=g)[:top] for _ in range(T)]).to(torch.int32).cuda()
    w = (torch.rand(T * top, generator=g) * 0.8 + 0.1).cuda()
    results = []
    for mma in (True, False):
        monkeypatch.setattr(ops, "MOE_MMA", mma)
        plan = ops.moe_plan(ids, E, ops.moe_row_tile(ops.moe_on_tensor_cores(torch.bfloat16, K, I), T * top, E))
        act = torch.zeros((T * top, I), dtype=torch.bfloat16, device="cuda")
        out = torch.zeros((T * top, K), dtype=torch.bfloat16, device="cuda")
        ops.moe_gate_up(x, w, plan, gate, up, act, top, 1.5, 1.702)
        ops.moe_down(act, plan, down, out)
        results.append((act.float().cpu(), out.float().cpu()))
    # against float64, pair by pair
    for pair in range(T * top):
        e, h = int(ids.view(-1)[pair]), x[pair // top].double().cpu() * float(w[pair])
        a = (gate[e].double().cpu() @ h).clamp(max=1.5)
        b = (up[e].double().cpu() @ h).clamp(-1.5, 1.5)
        want = down[e].double().cpu() @ (a * torch.sigmoid(1.702 * a) * (b + 1))
        for act, out in results:
            assert float((out[pair].double() - want).abs().max()) < 3e-2 * float(want.abs().max()) + 1e-3
    assert float((results[0][1] - results[1][1]).abs().max()) < 2e-2 * float(results[1][1].abs().max())
