"""Fegetar without a GPU: the configuration and registry, the tensor list, and properties of the
plain implementation that the GPU tests rely on as their yardstick."""

import copy
import math

import pytest
import torch

from tests.fegetar_configs import FEG, fegetar_weights, random_ids, tensor_shapes
from tests.plain import fegetar_plain as plain
from tokensprint_b200.config.model_config import ConfigError
from tokensprint_b200.config.registry import architecture_for


@pytest.mark.parametrize("tag", sorted(FEG))
def test_config_names_its_architecture_and_round_trips(tag):
    cfg = FEG[tag]
    arch = architecture_for(cfg)
    assert arch.name == "Fegetar"
    typed = arch.config_from_dict(cfg)
    assert typed.to_dict() == cfg
    assert arch.config_from_dict(typed.to_dict()) == typed


@pytest.mark.parametrize("tag", sorted(FEG))
def test_tensor_list_follows_the_config(tag):
    cfg = FEG[tag]
    arch = architecture_for(cfg)
    spec = arch.build_spec(arch.config_from_dict(cfg))
    assert {s.name: tuple(s.shape) for s in spec.tensor_specs()} == tensor_shapes(cfg)


def test_config_errors_name_the_key():
    arch = architecture_for(FEG["a"])
    for path, value, word in ((("layers", 0, "type"), "other", "type"), (("layers", 0, "mixer", "rot", "dims"), 7, "rot.dims"),
                              (("layers", 0, "mlp", "router", "top"), 9, "router.top"), (("norm", "eps"), 0.0, "norm.eps"),
                              (("layers", 1, "mlp", "kind"), "glu", "mlp.kind")):
        bad = copy.deepcopy(FEG["a"])
        d = bad
        for k in path[:-1]:
            d = d[k]
        d[path[-1]] = value
        with pytest.raises(ConfigError, match=word.replace(".", r"\.")):
            arch.config_from_dict(bad)
    missing = copy.deepcopy(FEG["a"])
    del missing["layers"][0]["mixer"]["kv_rank"]
    with pytest.raises(ConfigError, match="kv_rank"):
        arch.config_from_dict(missing)


def test_pair_rows():
    assert plain.pair_rows([5, 7, 7, 0], 31, 5, 97) == [97, (5 * 31 + 7 * 5) % 97, (7 * 31 + 7 * 5) % 97, (7 * 31) % 97]


def test_rotation_keeps_lengths_and_depends_on_distance_only():
    g = torch.Generator().manual_seed(0)
    q, k = torch.randn(1, 12, generator=g, dtype=torch.float64), torch.randn(1, 12, generator=g, dtype=torch.float64)
    a = plain.rotate_pairs(q, [40], 1000.0, 8)
    assert torch.allclose(a[:, 8:], q[:, 8:]) and torch.allclose(a[:, :8].norm(), q[:, :8].norm())
    dots = [float((plain.rotate_pairs(q, [p + 9], 1000.0, 8) * plain.rotate_pairs(k, [p], 1000.0, 8)).sum()) for p in (0, 3, 700)]
    assert max(dots) - min(dots) < 1e-9
    # neighbours are paired: entry 0 with 1, by the angle p * base^0 = p
    e = torch.zeros(1, 4, dtype=torch.float64)
    e[0, 0] = 1.0
    r = plain.rotate_pairs(e, [2], 50.0, 4)
    assert torch.allclose(r[0], torch.tensor([math.cos(2.0), math.sin(2.0), 0.0, 0.0], dtype=torch.float64))


def test_latent_attention_equals_scoring_the_latent_with_absorbed_queries():
    """The engine never rebuilds keys: it scores U_k^T q against the latent and applies U_v to the
    weighted sum of latents.  Both are the same function."""
    cfg = FEG["a"]
    m, eps = cfg["layers"][0]["mixer"], cfg["norm"]["eps"]
    W = {k: v.double() for k, v in fegetar_weights(cfg, 4).items()}
    T = 9
    h = torch.randn(T, cfg["width"], generator=torch.Generator().manual_seed(1), dtype=torch.float64)
    pos = list(range(T))
    want = plain.latent_attention(h, pos, W, "l0.mix.", m, eps)
    H, dn, dr, dv, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    q = (h @ W["l0.mix.q"].T).view(T, H, dn + dr)
    down = h @ W["l0.mix.dkv"].T
    c = plain.norm_plain(down[:, :R], W["l0.mix.dkv.norm"], eps)
    r = plain.rotate_pairs(down[:, R:], pos, m["rot"]["base"], m["rot"]["dims"])
    uk, uv = W["l0.mix.uk"].view(H, dn, R), W["l0.mix.uv"].view(H, dv, R)
    q_abs = torch.einsum("thd,hdr->thr", q[..., :dn], uk)
    q_rot = plain.rotate_pairs(q[..., dn:], pos, m["rot"]["base"], m["rot"]["dims"])
    s = (torch.einsum("thr,sr->hts", q_abs, c) + torch.einsum("thd,sd->hts", q_rot, r)) * m["scale"]
    s = s.masked_fill(torch.triu(torch.ones(T, T, dtype=torch.bool), 1)[None], float("-inf"))
    o = torch.einsum("hts,sr->thr", torch.softmax(s, -1), c)
    o = torch.einsum("thr,hvr->thv", o, uv) * torch.sigmoid(h @ W["l0.mix.g"].T)[..., None]
    assert torch.allclose(o.reshape(T, H * dv) @ W["l0.mix.o"].T, want, atol=1e-10)


def test_routing_weights_multiply_the_input_and_limits_bite():
    cfg = FEG["a"]
    mlp = cfg["layers"][0]["mlp"]
    W = {k: v.double() for k, v in fegetar_weights(cfg, 5).items()}
    h = torch.randn(6, cfg["width"], generator=torch.Generator().manual_seed(2), dtype=torch.float64)
    e, w = plain.route(h, W, "l0.mlp.", 2)
    assert e.shape == (6, 2) and bool((w[:, 0] >= w[:, 1]).all()) and bool(((w > 0) & (w < 1)).all())
    got = plain.routed_ff(h, W, "l0.mlp.", mlp)
    by_hand = plain.capped_expert(h, W, "l0.mlp.shared.", mlp["shared"]["limit"])
    for t in range(6):
        for j in range(2):
            by_hand[t] += plain.capped_expert(w[t, j] * h[t : t + 1], W, f"l0.mlp.e{int(e[t, j])}.", mlp["expert"]["limit"])[0]
    assert torch.allclose(got, by_hand, atol=1e-12)
    # the weight on the output would be another function (the expert is not linear)
    other = plain.capped_expert(h[:1], W, f"l0.mlp.e{int(e[0, 0])}.", mlp["expert"]["limit"])[0] * w[0, 0]
    mine = plain.capped_expert(w[0, 0] * h[:1], W, f"l0.mlp.e{int(e[0, 0])}.", mlp["expert"]["limit"])[0]
    assert not torch.allclose(other, mine, atol=1e-6)
    pre = (h @ W["l0.mlp.e0.gate"].T)
    assert float(pre.max()) > mlp["expert"]["limit"], "the test's weights never reach the limit"


@pytest.mark.parametrize("tag", sorted(FEG))
def test_plain_model_is_causal_and_its_first_token_takes_the_extra_row(tag):
    cfg = FEG[tag]
    W = fegetar_weights(cfg, 6)
    ids = random_ids(cfg, 14, 7)
    a, layers = plain.forward(ids, W, cfg)
    other = list(ids)
    other[9] = (other[9] + 1) % cfg["vocab"]
    b, _ = plain.forward(other, W, cfg)
    assert torch.equal(a[:9], b[:9]) and not torch.allclose(a[9:], b[9:])
    assert layers.shape == (len(cfg["layers"]), 14, cfg["width"])
    pair = (cfg.get("embedding") or {}).get("bigram")
    if pair:
        x = plain.embed(ids, W, cfg)
        assert torch.allclose(x[0], (W["embed"][ids[0]] + W["bigram"][pair["buckets"]]).double())
