"""Fegetar models of random shapes through the engine: widths, head counts, ranks and rotated parts
that are multiples of nothing in particular, layers of different shapes in one model, heads without
an unrotated part, rotations narrower than the rotated part or absent, one expert, as many experts
per token as there are experts, every optional piece present or absent.  Each model runs whole, in
portions, with a decoded tail and mixed with pages used again, in float32 against the float64 plain
model (sharpened queries), and in bfloat16 for finite logits that agree between the cuttings (what
bfloat16 rounding does to a random model of odd shape has no useful bound against float64)."""

import random

import numpy as np
import pytest

from tests.fegetar_configs import fegetar_weights, random_ids, write_fegetar_folder
from tests.plain import fegetar_plain as plain
from tests.replay_helpers import replay_in_process, trace_decode_tail, trace_mixed, trace_portions, trace_whole

pytestmark = pytest.mark.gpu


def random_config(rng: random.Random) -> dict:
    def mixer():
        dn, dr = rng.choice([0, 8, 16, 24, 32, 40, 64]), rng.choice([2, 4, 8, 16, 32, 48])
        dims = rng.choice(range(0, dr + 1, 2)) if rng.random() < 0.3 else dr
        return {"heads": rng.choice([1, 2, 3, 4, 6, 8, 16]), "dim": dn, "rot_dim": dr, "vdim": rng.choice([8, 12, 16, 32, 64]),
                "kv_rank": rng.choice([8, 16, 20, 32, 48, 64, 96, 128]), "scale": rng.choice([0.05, 0.1, 0.2]),
                "rot": {"base": rng.choice([100.0, 10000.0, 1e6]), "dims": dims}}

    width, same, first = rng.choice([40, 56, 64, 100, 128, 136, 200, 256, 320]), rng.random() < 0.6, None
    layers = []
    for _ in range(rng.randint(1, 5)):
        k = rng.random()
        if k < 0.2:
            mlp = None
        elif k < 0.55:
            mlp = {"kind": "dense", "ff": rng.choice([24, 64, 100, 256])}
        else:
            experts = rng.choice([1, 2, 4, 6, 12, 33])
            mlp = {"kind": "moe", "router": {"experts": experts, "top": rng.randint(1, min(experts, 4))},
                   "expert": {"ff": rng.choice([8, 24, 36, 64]), "limit": rng.choice([0.5, 2.0, 7.0])},
                   "shared": {"ff": rng.choice([16, 40, 96]), "limit": rng.choice([1.0, 3.0])} if rng.random() < 0.6 else None}
        first = first or mixer()
        layers.append({"type": "latent_attention", "mixer": first if same else mixer(), "mlp": mlp})
    cfg = {"architecture": "Fegetar", "vocab": rng.choice([50, 211, 333, 1000]), "width": width, "norm": {"eps": rng.choice([1e-5, 1e-6])}, "layers": layers}
    if rng.random() < 0.7:
        cfg["embedding"] = {"bigram": {"buckets": rng.choice([7, 97, 601, 4099]), "mul_prev": rng.choice([1, 31, 113, 1000003]), "mul_cur": rng.choice([1, 5, 13])}}
    if rng.random() < 0.7:
        cfg["token_side"] = {"dim": rng.choice([3, 8, 12, 20])}
    return cfg


@pytest.mark.parametrize("seed", range(8))
def test_random_model_in_every_cutting(tmp_path, seed):
    from tokensprint_b200.engine.replay import TraceReplayer

    cfg = random_config(random.Random(1000 + seed))
    requests = {f"r{i}": random_ids(cfg, n, seed * 100 + i) for i, n in enumerate([1, 7, 40, 90, 131])}
    for dtype, sharp in (("float32", 2.0), ("bfloat16", 1.0)):
        weights = fegetar_weights(cfg, seed, sharp=sharp, routed_share=1.0 if dtype == "float32" else 0.01)
        folder = write_fegetar_folder(tmp_path / dtype, cfg, weights)
        want = {k: plain.forward(v, weights, cfg)[0].numpy() for k, v in requests.items()}
        runs = {}
        for name, steps, max_tokens in (("whole", trace_whole(requests), 512), ("portions", trace_portions(requests), 512),
                                        ("tail", trace_decode_tail(requests, 8), 512), ("mixed", trace_mixed(requests, 320, seed=seed, max_live=3), 320)):
            replayer = TraceReplayer.from_folder(folder, dtype, max_tokens, page_size=16, max_live=3)
            replayer.runner.poison_freed_pages = True
            runs[name] = got = replay_in_process(replayer, steps)
            assert len(got) == sum(len(v) for v in requests.values())
            for (rid, pos), row in got.items():
                assert np.isfinite(row).all(), f"{dtype} {name}: request {rid} position {pos} is not finite"
                if dtype == "float32":
                    err = float(np.abs(row - want[rid][pos]).max() / np.abs(want[rid]).max())
                    assert err < 3e-4, f"float32 {name}: request {rid} position {pos}: error {err:.3g}\n{cfg}"
        tol = 1e-4 if dtype == "float32" else 5e-2
        for name in ("portions", "tail", "mixed"):
            for key, row in runs["whole"].items():
                scale = float(np.abs(want[key[0]]).max())
                assert float(np.abs(row - runs[name][key]).max()) <= tol * scale, f"{dtype}: whole and {name} differ at {key}\n{cfg}"
