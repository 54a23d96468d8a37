"""Host tests of the Dazilix design: the plain model against closed forms of its own mechanisms,
the typed configuration and the tensor names, the run order, and the cache manager's groups for
attention that sees blocks of positions."""

import math

import pytest
import torch

from tests.dazilix_configs import DAZ, DECAY_RANK, dazilix_weights, random_ids, tensor_shapes
from tests.plain import dazilix_plain as plain


def test_sink_softmax_is_a_softmax_with_one_more_key_of_score_zero():
    g = torch.Generator().manual_seed(1)
    scores = torch.randn(5, 9, generator=g, dtype=torch.float64) * 3
    visible = torch.rand(5, 9, generator=g) < 0.7
    visible[:, 0] = True
    got = plain.sink_softmax(scores, visible)
    padded = torch.cat([scores.masked_fill(~visible, -math.inf), torch.zeros(5, 1, dtype=torch.float64)], dim=1)
    want = torch.softmax(padded, dim=1)[:, :9]
    assert torch.allclose(got, want, atol=1e-14)
    assert (got.sum(1) < 1).all() and (got[~visible] == 0).all()


def test_block_mask_counts_blocks_from_position_zero():
    m = plain.block_mask(range(10), 4)
    assert m[3].tolist() == [True] * 4 + [False] * 6
    assert m[4].tolist() == [False] * 4 + [True] + [False] * 5  # the first position of a block sees itself alone
    assert m[7].tolist() == [False] * 4 + [True] * 4 + [False] * 2
    assert m[9].tolist() == [False] * 8 + [True] * 2
    shifted = plain.block_mask(range(6, 10), 4)  # positions 6..9 of a longer sequence: the edge stays at 8
    assert shifted.tolist() == [[True, False, False, False], [True, True, False, False], [False, False, True, False], [False, False, True, True]]


def test_rotation_turns_the_first_entries_and_keeps_lengths():
    g = torch.Generator().manual_seed(2)
    x = torch.randn(7, 3, 12, generator=g, dtype=torch.float64)
    y = plain.rotate_halves(x, range(7), 100.0, 8)
    assert torch.equal(y[..., 8:], x[..., 8:])
    assert torch.equal(y[0], x[0])  # position 0: no turn
    assert torch.allclose(y[..., :8].pow(2).sum(-1), x[..., :8].pow(2).sum(-1))
    a = 5 * 100.0 ** (-2 * 1 / 8)
    assert torch.allclose(y[5, 0, 1], x[5, 0, 1] * math.cos(a) - x[5, 0, 5] * math.sin(a))
    assert torch.allclose(y[5, 0, 5], x[5, 0, 5] * math.cos(a) + x[5, 0, 1] * math.sin(a))


def test_recurrence_equals_the_sum_over_earlier_tokens():
    """o_t = sum over s <= t of (q_t . (k_s * product of the decays after s)) v_s."""
    g = torch.Generator().manual_seed(3)
    T, d, e = 9, 5, 4
    q, k = torch.randn(T, d, generator=g, dtype=torch.float64), torch.randn(T, d, generator=g, dtype=torch.float64)
    v = torch.randn(T, e, generator=g, dtype=torch.float64)
    decay = torch.rand(T, d, generator=g, dtype=torch.float64) * 0.5 + 0.5
    out, state = plain.gla_recurrence(q, k, v, decay)
    for t in range(T):
        want = torch.zeros(e, dtype=torch.float64)
        for s in range(t + 1):
            shrink = decay[s + 1 : t + 1].prod(0)
            want += (q[t] * k[s] * shrink).sum() * v[s]
        assert torch.allclose(out[t], want, atol=1e-12)
    # cut in two: the state carries everything
    first, mid = plain.gla_recurrence(q[:4], k[:4], v[:4], decay[:4])
    second, end = plain.gla_recurrence(q[4:], k[4:], v[4:], decay[4:], mid)
    assert torch.allclose(torch.cat([first, second]), out, atol=1e-13) and torch.allclose(end, state, atol=1e-13)


def test_decay_is_the_sigmoid_to_the_power_one_over_tau():
    cfg = DAZ["b"]
    w = dazilix_weights(cfg, 5, decay_rank=DECAY_RANK["b"])
    m = cfg["layers"][0]["mixer"]
    h = torch.randn(4, cfg["width"], dtype=torch.float64)
    z = (h @ w["l0.mix.a1"].double().T) @ w["l0.mix.a2"].double().T + w["l0.mix.a2.b"].double()
    assert torch.allclose(plain.gla_decay(h, m, "l0.mix.", w), torch.sigmoid(z) ** (1.0 / m["tau"]), atol=1e-14)


def test_router_weights_are_the_softmax_over_the_chosen_logits():
    cfg = DAZ["a"]
    w = dazilix_weights(cfg, 6, decay_rank=DECAY_RANK["a"])
    f = cfg["layers"][3]["mlp"]
    h = torch.randn(11, cfg["width"], dtype=torch.float64)
    chosen, share = plain.route(h, f, "l3.mlp.", w)
    logits = h @ w["l3.mlp.router"].double().T + w["l3.mlp.router.b"].double()
    assert chosen.shape == (11, 3) and torch.allclose(share.sum(1), torch.ones(11, dtype=torch.float64))
    for t in range(11):
        order = torch.argsort(logits[t], descending=True)[:3]
        assert chosen[t].tolist() == order.tolist()
        assert torch.allclose(share[t], torch.softmax(logits[t][order], 0))
    one = dict(f, router=dict(f["router"], top=1))
    assert torch.equal(plain.route(h, one, "l3.mlp.", w)[1], torch.ones(11, 1, dtype=torch.float64))


def test_run_plan():
    assert plain.run_plan(DAZ["a"]) == [(0, None), (1, 0), (2, None), (1, 1), (2, None), (3, None)]
    assert plain.run_plan(DAZ["b"]) == [(0, None), (1, None)]
    assert plain.run_plan(DAZ["c"]) == [(0, 0), (1, None), (0, 1), (1, None), (0, 2), (1, None), (2, None)]


@pytest.mark.parametrize("tag", ["a", "b", "c"])
def test_logits_of_a_prefix_do_not_depend_on_what_follows(tag):
    cfg = DAZ[tag]
    w = dazilix_weights(cfg, 7, decay_rank=DECAY_RANK[tag])
    ids = random_ids(cfg, 45, 70)
    whole = plain.forward_logits(ids, w, cfg)
    assert torch.allclose(plain.forward_logits(ids[:19], w, cfg), whole[:19], atol=1e-10)


# ---------------------------------------------------------------------------
# the engine's configuration, registry and run order (no GPU needed)


@pytest.mark.parametrize("tag", ["a", "b", "c", "d"])
def test_config_and_tensor_names(tag):
    from tokensprint_b200.config.registry import architecture_for

    cfg = DAZ[tag]
    arch = architecture_for(cfg)
    typed = arch.config_from_dict(cfg)
    assert typed.to_dict() == cfg
    spec = arch.build_spec(typed)
    want = tensor_shapes(cfg, DECAY_RANK[tag])
    got = {s.name: tuple(s.shape) for s in spec.tensor_specs()}
    assert set(got) == set(want)
    for name, shape in got.items():
        assert all(g in (-1, w) for g, w in zip(shape, want[name])) and len(shape) == len(want[name]), name
    assert [(r.layer, None if r.before is None else spec.run_transforms[r.before].params["row"]) for r in spec.run_order] == plain.run_plan(cfg)
    assert [spec.run_transforms[r.before].params["add_embedding"] for r in spec.run_order if r.before is not None] == \
        [t > 0 for t in range(len(spec.run_transforms))]


def test_config_errors_name_the_key():
    from tokensprint_b200.config.model_config import ConfigError
    from tokensprint_b200.models.dazilix import DazilixConfig

    import copy

    for path, value in ((("layers", 0, "type"), "conv"), (("layers", 0, "mixer", "vdim"), 8), (("layers", 0, "mixer", "rot", "dims"), 7),
                        (("loop", "stop"), 9), (("layers", 0, "mlp", "router", "top"), 0), (("layers", 1, "mixer", "tau"), 0.0)):
        bad = copy.deepcopy(DAZ["a"])
        node = bad
        for key in path[:-1]:
            node = node[key]
        node[path[-1]] = value
        with pytest.raises(ConfigError):
            DazilixConfig.from_dict(bad)


def test_random_weights_need_the_decay_rank():
    from tokensprint_b200.config.registry import architecture_for
    from tokensprint_b200.weights.loader import RandomSource

    cfg = DAZ["b"]
    arch = architecture_for(cfg)
    with pytest.raises(ValueError, match="a1"):
        RandomSource(arch.build_spec(arch.config_from_dict(cfg)).tensor_specs(), 1)
    import copy

    named = copy.deepcopy(cfg)
    for layer in named["layers"]:
        layer["mixer"]["decay_rank"] = 4
    typed = arch.config_from_dict(named)
    assert typed.to_dict() == named
    shapes = RandomSource(arch.build_spec(typed).tensor_specs(), 1).shapes()
    assert shapes["l0.mix.a1"] == (4, cfg["width"]) and shapes["l1.mix.a2"] == (6 * 36, 4)


def test_chunk_group_gives_back_the_pages_of_earlier_blocks():
    from tokensprint_b200.cache.manager import CacheManager, GroupSpec

    cm = CacheManager([GroupSpec("chunk", 24), GroupSpec("full")], page_size=8, pages_per_group=[6, 12], num_slots=2)
    rc = cm.admit("r")
    cm.extend(rc, 0, 30)  # positions 0..29: the query at 29 sees 24..29, but the step's first query (0) sees 0
    assert cm.pages_in_use(0) == 4 and cm.pages_in_use(1) == 4
    cm.extend(rc, 30, 31)  # a query at 30: its block began at 24, pages 0..2 go
    assert rc.tables[0][:3] == [-1, -1, -1] and cm.pages_in_use(0) == 1 and cm.pages_in_use(1) == 4
    cm.extend(rc, 31, 48)  # up to position 47, still the block of 24..47
    assert cm.pages_in_use(0) == 3
    cm.extend(rc, 48, 49)  # position 48 opens a block: nothing before it is seen again
    assert cm.pages_in_use(0) == 1 and cm.pages_in_use(1) == 7
    cm.check_invariants()
    cm.free(rc)
    assert cm.pages_in_use(0) == 0 and cm.pages_in_use(1) == 0
