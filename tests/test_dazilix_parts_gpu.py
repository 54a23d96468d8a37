"""Each mechanism of the Dazilix design alone: the engine's kernels against the plain functions of
tests/plain/dazilix_plain.py, on made-up inputs where random ones would hide a fault (a far key
that stands out, keys just inside and just outside a block of positions, a sink that matters)."""

import math

import pytest
import torch

from tests.plain import dazilix_plain as plain

pytestmark = pytest.mark.gpu

DEV = "cuda"
TOL = {torch.float32: 2e-5, torch.bfloat16: 2e-2}


def _randn(*shape, seed=0, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(*shape, generator=g, dtype=torch.float64) * scale


def _rel(got: torch.Tensor, want: torch.Tensor) -> float:
    return float((got.double().cpu() - want).abs().max() / want.abs().max().clamp_min(1e-30))


# ---------------------------------------------------------------------------
# attention inside blocks of positions, with a sink


def _paged(rows: torch.Tensor, page: int, dtype, seed: int):
    """rows [n, heads, d] of one sequence -> (pool [pages, page, heads, d] with the pages in a shuffled order, table)."""
    n = rows.shape[0]
    pages = -(-n // page)
    g = torch.Generator().manual_seed(seed)
    order = torch.randperm(pages + 3, generator=g)[:pages]
    pool = torch.full((pages + 3, page, *rows.shape[1:]), float("nan"), dtype=torch.float64)
    for j in range(n):
        pool[order[j // page], j % page] = rows[j]
    return pool.to(dtype).to(DEV), order.to(torch.int32)


def _attend(kernel, q, k, v, positions, page, nq, nkv, d, scale, chunk, sink, dtype):
    """One sequence: queries at `positions` against keys 0..len(k)-1 through the paged kernel."""
    from tokensprint_b200 import ops

    T = q.shape[0]
    kp, table = _paged(k, page, dtype, 11)
    vp, _ = _paged(v, page, dtype, 11)
    out = torch.empty((T, nq * d), device=DEV, dtype=dtype)
    pos = torch.tensor(list(positions), dtype=torch.int32, device=DEV)
    seq = torch.zeros(T, dtype=torch.int32, device=DEV)
    qd = q.reshape(T, nq * d).to(dtype).to(DEV)
    if kernel == "simple":
        ops.attention_paged_simple(qd, kp, vp, out, pos, seq, table.view(1, -1).to(DEV), page, nq, nkv, d, scale, 0, chunk, sink)
    elif kernel == "tcgen05":
        cu = torch.tensor([0, T], dtype=torch.int32, device=DEV)
        lens = torch.tensor([positions[-1] + 1], dtype=torch.int32, device=DEV)
        ops.attention_prefill_tcgen05(qd, kp, vp, out, cu, lens, table.view(1, -1).to(DEV), page, 1, T, nq, nkv, scale, 0, chunk=chunk, sink=sink)
        ops.check_device_errors()
    else:
        cu = torch.tensor([0, T], dtype=torch.int32, device=DEV)
        lens = torch.tensor([positions[-1] + 1], dtype=torch.int32, device=DEV)
        ops.attention_paged_mma(qd, kp, vp, out, cu, lens, table.view(1, -1).to(DEV), seq, page, 1, T, nq, nkv, d, scale, 0, 1, None, 0,
                                chunk=chunk, sink=sink)
    torch.cuda.synchronize()
    return out.view(T, nq, d)


def _plain_attend(q, k, v, positions, nq, nkv, scale, chunk, sink):
    T, n = q.shape[0], k.shape[0]
    p = torch.as_tensor(list(positions))
    keys = torch.arange(n)
    visible = keys[None, :] <= p[:, None]
    if chunk:
        visible &= (keys[None, :] // chunk) == (p[:, None] // chunk)
    out = torch.empty(T, nq, q.shape[-1], dtype=torch.float64)
    for h in range(nq):
        s = (q[:, h] @ k[:, h // (nq // nkv)].T) * scale
        if sink:
            w = plain.sink_softmax(s, visible)
        else:
            w = torch.softmax(s.masked_fill(~visible, -math.inf), dim=-1)
        out[:, h] = w @ v[:, h // (nq // nkv)]
    return out


KERNELS = ["simple", "mma"]


@pytest.mark.parametrize("kernel", KERNELS)
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nq, nkv, d, chunk, page", [(4, 2, 32, 16, 16), (6, 6, 16, 8, 16), (5, 1, 48, 40, 16), (2, 2, 64, 24, 8), (3, 1, 64, 64, 32)])
def test_block_attention_with_sink_random(kernel, dtype, nq, nkv, d, chunk, page):
    if kernel == "mma" and dtype == torch.float32:
        pytest.skip("the tensor-core kernel is bfloat16 only")
    n = 150
    q, k, v = _randn(n, nq, d, seed=1), _randn(n, nkv, d, seed=2), _randn(n, nkv, d, seed=3)
    q, k, v = (x.to(dtype).double() for x in (q, k, v))
    scale = 0.4 * d ** -0.5 * 3
    want = _plain_attend(q, k, v, range(n), nq, nkv, scale, chunk, True)
    # a whole prompt, a portion that starts inside a block, single decoded tokens at and around an edge
    for positions in (range(n), range(chunk + 3, min(n, 3 * chunk + 5)), [2 * chunk - 1], [2 * chunk], [2 * chunk + 1], [n - 1]):
        positions = list(positions)
        got = _attend(kernel, q[positions], k[: positions[-1] + 1], v[: positions[-1] + 1], positions, page, nq, nkv, d, scale, chunk, 0.0, dtype)
        assert _rel(got, want[positions]) < TOL[dtype], (positions[0], positions[-1])


@pytest.mark.parametrize("kernel", ["mma", "tcgen05"])
@pytest.mark.parametrize("nq, nkv, chunk, page", [(4, 2, 48, 16), (8, 1, 100, 16), (2, 2, 256, 64), (5, 1, 64, 8)])
def test_block_attention_with_sink_heads_of_128(kernel, nq, nkv, chunk, page):
    """Heads of 128, where prompt portions run on the tcgen05 kernel: portions of more rows than one
    tile of 128 (two tiles per CTA) and of fewer, starting inside a block, with and without a sink."""
    from tokensprint_b200 import ops

    d, n, dtype = 128, 330, torch.bfloat16
    if kernel == "tcgen05" and not ops.attention_tcgen05_supported(nq, nkv, d, page):
        pytest.skip("sizes the tcgen05 kernel does not take")
    q, k, v = (_randn(n, h, d, seed=s).to(dtype).double() for h, s in ((nq, 11), (nkv, 12), (nkv, 13)))
    scale = 0.1
    for sink in (0.0, None):
        want = _plain_attend(q, k, v, range(n), nq, nkv, scale, chunk, sink is not None)
        for positions in (range(n), range(chunk + 3, chunk + 3 + 21), range(min(2 * chunk, n - 30) - 7, n), range(5)):
            positions = list(positions)
            got = _attend(kernel, q[positions], k[: positions[-1] + 1], v[: positions[-1] + 1], positions, page, nq, nkv, d, scale, chunk, sink, dtype)
            assert _rel(got, want[positions]) < TOL[dtype], (sink, positions[0], positions[-1])


@pytest.mark.parametrize("kernel", KERNELS)
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_block_edges_and_far_keys_show(kernel, dtype):
    """One key carries nearly all of a query's weight.  Just inside the block (its first position, far
    from the query) it must be found; just outside (the position before the block) it must not."""
    if kernel == "mma" and dtype == torch.float32:
        pytest.skip("the tensor-core kernel is bfloat16 only")
    nq, nkv, d, chunk, page = 2, 1, 32, 48, 16
    n = 4 * chunk
    q, k, v = _randn(n, nq, d, seed=4, scale=0.1), _randn(n, nkv, d, seed=5, scale=0.1), _randn(n, nkv, d, seed=6)
    direction = torch.zeros(d, dtype=torch.float64)
    direction[3] = 1.0
    for query, key in ((3 * chunk - 1, 2 * chunk), (3 * chunk - 1, 2 * chunk - 1), (3 * chunk, 3 * chunk - 1), (3 * chunk + 1, 3 * chunk),
                       (chunk - 1, 0), (chunk, 0)):
        kk, qq = k.clone(), q.clone()
        kk[key, 0], qq[query, :] = 8.0 * direction, 8.0 * direction
        qq, kk, vv = (x.to(dtype).double() for x in (qq, kk, v))
        for positions in ([query], list(range(query - 5, query + 1))):
            got = _attend(kernel, qq[positions], kk[: query + 1], vv[: query + 1], positions, page, nq, nkv, d, 1.0, chunk, 0.0, dtype)
            want = _plain_attend(qq, kk, vv, range(n), nq, nkv, 1.0, chunk, True)[positions]
            inside = key // chunk == query // chunk
            hit = float((got[-1, 0].double().cpu() - vv[key, 0]).abs().max())
            assert (hit < 0.05) == inside, f"query {query}, key {key}: the key is {'inside' if inside else 'outside'} the block"
            assert _rel(got, want) < TOL[dtype], (query, key)


@pytest.mark.parametrize("cluster", [True, False])
@pytest.mark.parametrize("d, nq, nkv", [(64, 4, 2), (128, 8, 1), (32, 2, 2)])
def test_decode_with_the_keys_split_over_ctas_keeps_bound_and_sink(d, nq, nkv, cluster):
    """Single decoded tokens of three sequences of unequal length, the keys of each cut into 1 to 8
    ranges that separate CTAs take and a merge puts together (inside a thread-block cluster, or by a
    second kernel): the sink must be counted once, whichever range is empty, and the block bound hold."""
    from tokensprint_b200 import ops

    page, dtype, scale = 16, torch.bfloat16, 0.2
    lens = [700, 37, 300]
    B = len(lens)
    ops._attention_mma_fns(d)  # loads the library of this head size, so that its merge mode can be set below
    for chunk in (0, 256, 48):
        for sink in (0.0, None, 1.5):
            qs, want, pools_k, pools_v, tables = [], [], [], [], []
            base = 0
            for b, n in enumerate(lens):
                q, k, v = (_randn(n, h, d, seed=100 * b + s).to(dtype).double() for h, s in ((nq, 1), (nkv, 2), (nkv, 3)))
                ref = _plain_attend(q, k, v, range(n), nq, nkv, scale, chunk, False) if sink is None else None
                if sink is not None:  # a sink of any score: one more key of that score whose value is zero
                    p = torch.arange(n)
                    visible = p[None, :] <= p[:, None]
                    if chunk:
                        visible &= (p[None, :] // chunk) == (p[:, None] // chunk)
                    ref = torch.empty(n, nq, d, dtype=torch.float64)
                    for h in range(nq):
                        sc = (q[:, h] @ k[:, h // (nq // nkv)].T) * scale
                        sc = torch.cat([sc.masked_fill(~visible, -math.inf), torch.full((n, 1), sink, dtype=torch.float64)], dim=1)
                        ref[:, h] = torch.softmax(sc, dim=1)[:, :n] @ v[:, h // (nq // nkv)]
                qs.append(q[n - 1])
                want.append(ref[n - 1])
                kp, table = _paged(k, page, dtype, 20 + b)
                vp, _ = _paged(v, page, dtype, 20 + b)
                pools_k.append(kp)
                pools_v.append(vp)
                tables.append(table + base)
                base += kp.shape[0]
            kpool, vpool = torch.cat(pools_k), torch.cat(pools_v)
            width = max(len(t) for t in tables)
            table = torch.full((B, width), -1, dtype=torch.int32)
            for b, t in enumerate(tables):
                table[b, : len(t)] = t
            qd = torch.stack(qs).reshape(B, nq * d).to(dtype).to(DEV)
            cu = torch.arange(B + 1, dtype=torch.int32, device=DEV)
            ctx = torch.tensor(lens, dtype=torch.int32, device=DEV)
            seq = torch.arange(B, dtype=torch.int32, device=DEV)
            for splits in (1, 2, 5, 8):
                out = torch.empty((B, nq * d), device=DEV, dtype=dtype)
                scratch = torch.empty(ops.attention_scratch_floats(B * nq, splits, d), device=DEV, dtype=torch.float32) if splits > 1 else None
                ops._attention_flat[d].ts_attention_mma_set_cluster_merge(1 if cluster else 0) if d in ops._attention_flat else None
                ops.attention_paged_mma(qd, kpool, vpool, out, cu, ctx, table.to(DEV), seq, page, B, 1, nq, nkv, d, scale, 0, splits, scratch, 0,
                                        chunk=chunk, sink=sink)
                if d in ops._attention_flat:
                    ops._attention_flat[d].ts_attention_mma_set_cluster_merge(1 if ops.ATTENTION_CLUSTER_MERGE else 0)
                torch.cuda.synchronize()
                assert _rel(out.view(B, nq, d), torch.stack(want)) < TOL[dtype], (chunk, sink, splits)


@pytest.mark.parametrize("kernel", KERNELS)
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_sink_takes_its_share(kernel, dtype):
    """All scores far below zero: the sink holds nearly all the weight and the output is nearly zero;
    without it the same scores give a plain average."""
    if kernel == "mma" and dtype == torch.float32:
        pytest.skip("the tensor-core kernel is bfloat16 only")
    nq, nkv, d, page = 2, 2, 32, 16
    n = 40
    k = torch.ones(n, nkv, d, dtype=torch.float64)
    q = -torch.ones(n, nq, d, dtype=torch.float64)
    v = _randn(n, nkv, d, seed=7) + 2.0
    v = v.to(dtype).double()
    for sink in (0.0, None, -4.0):
        got = _attend(kernel, q, k, v, range(n), page, nq, nkv, d, 0.25, 0, sink, dtype)
        s = -0.25 * d
        for t in (0, 7, n - 1):
            mean = v[: t + 1, 0].mean(0)
            share = 1.0 if sink is None else (t + 1) * math.exp(s) / ((t + 1) * math.exp(s) + math.exp(sink))
            assert float((got[t, 0].double().cpu() - share * mean).abs().max()) < TOL[dtype] * 4, (sink, t)


# ---------------------------------------------------------------------------
# q/k norm over the whole projection, rotation, store; values are the keys as projected


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nq, nkv, d, rot", [(4, 2, 24, 8), (6, 6, 16, 16), (5, 1, 12, 0), (2, 2, 64, 32), (3, 1, 10, 4)])
def test_joint_norm_rotation_and_store(dtype, nq, nkv, d, rot):
    from tokensprint_b200 import ops

    T, eps, base, pad = 9, 1e-5, 500.0, 5
    positions = [0, 1, 2, 40, 41, 1000, 1001, 7, 8]
    raw = _randn(T, (nq + nkv) * d + pad, seed=8).to(dtype)
    qk = raw.to(DEV)[:, : (nq + nkv) * d]  # a view with a longer row stride, as a slice of a wider product would be
    wq, wk = 1.0 + 0.2 * _randn(nq * d, seed=9), 1.0 + 0.2 * _randn(nkv * d, seed=10)
    slots = torch.tensor([3, 17, 4, -1, 9, 0, 21, 22, 8], dtype=torch.int32)
    q_out = torch.empty((T, nq * d), device=DEV, dtype=dtype)
    kc = torch.zeros((24, nkv, d), device=DEV, dtype=dtype)
    vc = torch.zeros_like(kc)
    cos_sin = None
    if rot:
        i = torch.arange(rot // 2, dtype=torch.float64)
        inv = (torch.tensor(base, dtype=torch.float64) ** (-2 * i / rot)).float().to(DEV)
        cos_sin = ops.rope_cos_sin(torch.tensor(positions, dtype=torch.int32, device=DEV), inv, T)
    ops.qk_joint_norm_rope_store(qk, q_out, kc, vc, slots.to(DEV), wq.float().to(DEV), wk.float().to(DEV), eps, cos_sin, nq, nkv, d)
    torch.cuda.synchronize()
    x = raw.double()
    qf, kf = x[:, : nq * d], x[:, nq * d : (nq + nkv) * d]
    want_q = plain.rotate_halves(plain.norm(qf, wq.float().double(), eps).reshape(T, nq, d), positions, base, rot)
    want_k = plain.rotate_halves(plain.norm(kf, wk.float().double(), eps).reshape(T, nkv, d), positions, base, rot)
    # positions near 1000 in float32 angles: an error of 1e-4 rad is rounding, a wrong pairing or frequency is of order one
    tol = max(TOL[dtype], 3e-4)
    assert _rel(q_out.view(T, nq, d), want_q) < tol
    for t in range(T):
        if slots[t] < 0:
            continue
        assert _rel(kc[slots[t]], want_k[t]) < tol
        assert torch.equal(vc[slots[t]].cpu(), raw[t, nq * d : (nq + nkv) * d].view(nkv, d)), "values are the key projection as it comes"
    untouched = [s for s in range(24) if s not in slots.tolist()]
    assert float(kc[untouched].abs().max()) == 0 and float(vc[untouched].abs().max()) == 0


# ---------------------------------------------------------------------------
# gated linear attention


def _gla_inputs(T, H, d, e, dtype, seed):
    q, k = _randn(T, H * d, seed=seed), _randn(T, H * d, seed=seed + 1)
    v, z = _randn(T, H * e, seed=seed + 2), _randn(T, H * d, seed=seed + 3, scale=2.0)
    bias = 1.0 + _randn(H * d, seed=seed + 4)
    return [x.to(dtype) for x in (q, k, v, z)] + [bias.float()]


def _plain_gla(q, k, v, z, bias, tau, q_scale, H, d, e, state=None):
    T = q.shape[0]
    decay = torch.exp(torch.nn.functional.logsigmoid(z.double() + bias.double()) / tau).reshape(T, H, d)
    out = torch.empty(T, H, e, dtype=torch.float64)
    new_state = torch.empty(H, d, e, dtype=torch.float64)
    for h in range(H):
        out[:, h], new_state[h] = plain.gla_recurrence(q.double().reshape(T, H, d)[:, h] * q_scale, k.double().reshape(T, H, d)[:, h],
                                                        v.double().reshape(T, H, e)[:, h], decay[:, h], None if state is None else state[h])
    return out.reshape(T, H * e), new_state


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H, d, e", [(1, 7, 10), (3, 20, 28), (2, 48, 64), (2, 128, 40), (1, 300, 33), (4, 64, 128)])
def test_gla_scan_unequal_sequences_and_portions(dtype, H, d, e):
    """Three sequences of unequal length in one batch, then each once more in portions (down to two
    tokens and to one) with the state carried in its slot; a slot is used again by another sequence."""
    from tokensprint_b200 import ops

    lens, tau, q_scale = [37, 1, 12], 6.0, d ** -0.5
    T = sum(lens)
    q, k, v, z, bias = _gla_inputs(T, H, d, e, dtype, 20)
    # q, k, v as columns of one wider matrix (one product's result), z on its own
    wide = torch.cat([q, k, v, torch.zeros(T, 3, dtype=dtype)], dim=1).to(DEV)
    qd, kd, vd = wide[:, : H * d], wide[:, H * d : 2 * H * d], wide[:, 2 * H * d : 2 * H * d + H * e]
    zd, bd = z.to(DEV), bias.to(DEV)
    state = torch.zeros((5, H, d, e), device=DEV, dtype=torch.float32)
    slots = torch.tensor([4, 0, 2], dtype=torch.int32, device=DEV)
    cu = torch.tensor([0, 37, 38, 50], dtype=torch.int32, device=DEV)
    out = torch.empty((T, H * e), device=DEV, dtype=torch.float32)
    ops.gla_scan(qd, kd, vd, zd, bd, tau, q_scale, state, slots, cu, out, 3, H, d, e)
    torch.cuda.synchronize()
    tol = 5e-5 if dtype == torch.float32 else 5e-5  # the inputs are read exactly in both types; the recurrence is float32
    start = 0
    finals = []
    for b, n in enumerate(lens):
        sl = slice(start, start + n)
        want, final = _plain_gla(q[sl], k[sl], v[sl], z[sl], bias, tau, q_scale, H, d, e)
        assert _rel(out[sl], want) < tol, f"sequence {b}"
        assert _rel(state[int(slots[b])], final) < tol, f"state of sequence {b}"
        finals.append((want, final))
        start += n
    assert float(state[1].abs().max()) == 0 and float(state[3].abs().max()) == 0, "a slot of no sequence was touched"
    # the first sequence again, in portions, in a slot that held another sequence (zeroed as the engine does on admission)
    state[2].zero_()
    done = 0
    for size in (5, 2, 1, 16, 2, 11):
        cu1 = torch.tensor([0, size], dtype=torch.int32, device=DEV)
        part = torch.empty((size, H * e), device=DEV, dtype=torch.float32)
        sl = slice(done, done + size)
        ops.gla_scan(qd[sl], kd[sl], vd[sl], zd[sl], bd, tau, q_scale, state, torch.tensor([2], dtype=torch.int32, device=DEV), cu1, part, 1, H, d, e)
        assert _rel(part, finals[0][0][sl]) < tol, f"portion at {done}"
        done += size
    assert done == 37 and _rel(state[2], finals[0][1]) < tol
    # a padded lane (no tokens) leaves its slot alone
    before = state.clone()
    ops.gla_scan(qd[:1], kd[:1], vd[:1], zd[:1], bd, tau, q_scale, state, torch.tensor([1, 3], dtype=torch.int32, device=DEV),
                 torch.tensor([0, 1, 1], dtype=torch.int32, device=DEV), torch.empty((1, H * e), device=DEV, dtype=torch.float32), 2, H, d, e)
    torch.cuda.synchronize()
    assert torch.equal(state[3], before[3]) and not torch.equal(state[1], before[1])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H, d, e", [(2, 20, 28), (1, 64, 128), (2, 7, 10)])
def test_gla_scan_long_portions_in_segments(dtype, H, d, e):
    """Portions long enough to be cut into segments that run side by side, beside a short one and a
    single token, each starting from a state that is not zero: against the plain recurrence, and
    against the same tokens run in one piece."""
    from tokensprint_b200 import ops

    lens, tau, q_scale = [1300, 5, 1, 700], 9.0, d ** -0.5
    T = sum(lens)
    q, k, v, z, bias = _gla_inputs(T, H, d, e, dtype, 40)
    wide = torch.cat([q, k, v], dim=1).to(DEV)
    qd, kd, vd = wide[:, : H * d], wide[:, H * d : 2 * H * d], wide[:, 2 * H * d :]
    zd, bd = z.to(DEV), (bias + 2.0).to(DEV)  # decays near one: what a segment starts from matters to its end
    start = (0.3 * _randn(6, H, d, e, seed=41)).float()
    slots = torch.tensor([5, 0, 3, 2], dtype=torch.int32, device=DEV)
    cu = torch.tensor([0, 1300, 1305, 1306, 2006], dtype=torch.int32, device=DEV)
    results = []
    for max_seqlen in (max(lens), None):
        assert (ops.gla_segments(4, max_seqlen)[0] > 1) == (max_seqlen is not None)
        state = start.clone().to(DEV)
        out = torch.empty((T, H * e), device=DEV, dtype=torch.float32)
        ops.gla_scan(qd, kd, vd, zd, bd, tau, q_scale, state, slots, cu, out, 4, H, d, e, max_seqlen=max_seqlen)
        torch.cuda.synchronize()
        results.append((out, state))
    begin = 0
    for b, n in enumerate(lens):
        sl = slice(begin, begin + n)
        want, final = _plain_gla(q[sl], k[sl], v[sl], z[sl], bias + 2.0, tau, q_scale, H, d, e, state=start[int(slots[b])].double())
        for out, state in results:
            assert _rel(out[sl], want) < 5e-5, f"sequence {b}"
            assert _rel(state[int(slots[b])], final) < 5e-5, f"state of sequence {b}"
        begin += n
    assert torch.equal(results[0][1][1].cpu(), start[1]) and torch.equal(results[0][1][4].cpu(), start[4]), "a slot of no sequence was touched"


def test_gla_state_remembers_a_far_token():
    """Decays of one on one key channel: a value written 600 tokens ago is read back exactly by a
    query on that channel; a channel whose decay is small has forgotten it."""
    from tokensprint_b200 import ops

    H, d, e, T = 1, 16, 8, 601
    q, k, v = torch.zeros(T, d), torch.zeros(T, d), torch.zeros(T, e)
    z = torch.full((T, d), -2.0)
    z[:, 5] = 40.0  # sigmoid = 1 in float32: this channel never forgets
    k[0, 5], k[0, 6] = 1.0, 1.0
    v[0] = torch.arange(1, e + 1, dtype=torch.float32)
    q[T - 1, 5] = 1.0
    q[T - 2, 6] = 1.0
    state = torch.zeros((1, H, d, e), device=DEV)
    out = torch.empty((T, e), device=DEV)
    wide = torch.cat([q, k, v], dim=1).to(DEV)
    ops.gla_scan(wide[:, :d], wide[:, d : 2 * d], wide[:, 2 * d :], z.to(DEV), None, 2.0, 1.0, state, torch.zeros(1, dtype=torch.int32, device=DEV),
                 torch.tensor([0, T], dtype=torch.int32, device=DEV), out, 1, H, d, e)
    torch.cuda.synchronize()
    assert torch.allclose(out[T - 1].cpu(), v[0], atol=1e-6)
    assert float(out[T - 2].abs().max()) < 1e-6


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H, e", [(1, 10), (3, 28), (4, 128)])
def test_gla_head_norm_and_gate(dtype, H, e):
    from tokensprint_b200 import ops

    T, eps = 6, 1e-5
    o = _randn(T, H * e, seed=30, scale=5.0).float()
    gate = _randn(T, H * e + 4, seed=31).to(dtype)
    w = (1.0 + 0.2 * _randn(e, seed=32)).float()
    out = torch.empty((T, H * e), device=DEV, dtype=dtype)
    ops.gla_norm_gate(o.to(DEV), gate.to(DEV)[:, : H * e], w.to(DEV), out, H, e, eps)
    torch.cuda.synchronize()
    want = plain.norm(o.double().reshape(T, H, e), w.double(), eps).reshape(T, H * e) * plain.silu(gate.double()[:, : H * e])
    assert _rel(out, want) < TOL[dtype]


# ---------------------------------------------------------------------------
# routed SwiGLU experts


@pytest.mark.parametrize("E, top", [(5, 2), (3, 1), (40, 4), (4, 4)])
def test_router_softmax_over_the_chosen_logits(E, top):
    from tokensprint_b200 import ops

    T, W = 33, 72
    x = _randn(T, W, seed=40).float()
    router = (_randn(E, W, seed=41) / W ** 0.5 * 2).float()
    bias = (0.5 * _randn(E, seed=42)).float()
    ids = torch.empty((T, top), dtype=torch.int32, device=DEV)
    weights = torch.empty((T, top), dtype=torch.float32, device=DEV)
    ops.router(x.to(DEV), router.to(DEV), top, False, ids, weights, bias=bias.to(DEV), score="softmax_chosen")
    logits = x.double() @ router.double().T + bias.double()
    want = torch.topk(logits, top, dim=-1)
    assert torch.equal(ids.cpu().long(), want.indices)
    assert torch.allclose(weights.cpu().double(), torch.softmax(want.values, -1), atol=2e-6)
    # the bias decides: a large bias on the last expert puts it first everywhere
    bias2 = bias.clone()
    bias2[E - 1] = 50.0
    ops.router(x.to(DEV), router.to(DEV), top, False, ids, weights, bias=bias2.to(DEV), score="softmax_chosen")
    assert (ids[:, 0].cpu() == E - 1).all()
    # the same choice from given logits
    ops.router_topk(logits.float().to(DEV) - bias.to(DEV), top, False, ids, weights, bias=bias.to(DEV), score="softmax_chosen")
    assert torch.allclose(weights.cpu().double(), torch.softmax(want.values, -1), atol=1e-5)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T, W, I, E, top", [(19, 72, 20, 3, 1), (70, 96, 40, 5, 2), (300, 64, 48, 9, 3), (5, 50, 24, 4, 4)])
def test_routed_swiglu_experts(dtype, T, W, I, E, top):
    """The whole feed-forward part against the plain one (the router reads the same rounded rows)."""
    from tokensprint_b200.parts.base import BuildContext, PartSpec, build_part

    ctx = BuildContext(device=torch.device(DEV), dtype=dtype)
    part = build_part("feed_forward", PartSpec("routed_experts", {
        "hidden_size": W, "num_experts": E, "top": top, "intermediate_size": I, "activation": "swiglu", "score": "softmax_chosen",
        "weight_on": "output", "router": "r", "router_bias": "r.b", "expert_prefix": "e"}), ctx)
    weights = {"r": (_randn(E, W, seed=50) / W ** 0.5 * 2), "r.b": 0.5 * _randn(E, seed=51)}
    for e in range(E):
        weights[f"e{e}.gate"] = _randn(I, W, seed=60 + 3 * e) / W ** 0.5 * 2
        weights[f"e{e}.up"] = _randn(I, W, seed=61 + 3 * e) / W ** 0.5
        weights[f"e{e}.down"] = _randn(W, I, seed=62 + 3 * e) / I ** 0.5
    weights = {k: v.to(torch.bfloat16).double() for k, v in weights.items()}
    roles = {s.name: s.role for s in part.tensor_specs()}
    part.load({k: v.to(DEV, torch.float32 if roles[k] == "vector" else dtype) for k, v in weights.items()})
    x = _randn(T, W, seed=52).to(dtype)
    got = part.forward(x.to(DEV), None)
    torch.cuda.synchronize()
    want = plain.routed_feed_forward(x.double(), {"router": {"top": top}}, "", {("router" if k == "r" else "router.b" if k == "r.b" else k): v
                                                                               for k, v in weights.items()})
    assert _rel(got, want) < (1e-5 if dtype == torch.float32 else 3e-2)


# ---------------------------------------------------------------------------
# the norms around a sublayer, the scale, the stream


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("W", [72, 96, 2048, 5000])
def test_branch_norm_scale_add_and_next_norm(dtype, W):
    from tokensprint_b200 import ops

    T, eps, eps2 = 7, 1e-5, 3e-6
    branch = _randn(T, W, seed=70, scale=3.0).to(dtype)
    hidden = _randn(T, W, seed=71).float()
    w, s, w2 = ((1.0 + 0.2 * _randn(W, seed=72 + i)).float() for i in range(3))
    want_h = hidden.double() + plain.norm(branch.double(), w.double(), eps) * s.double()
    want_x = plain.norm(want_h, w2.double(), eps2)
    h1 = hidden.clone().to(DEV)
    ops.branch_norm_add(branch.to(DEV), w.to(DEV), s.to(DEV), h1, eps)
    assert _rel(h1, want_h) < 1e-6
    h2 = hidden.clone().to(DEV)
    out = torch.empty((T, W), device=DEV, dtype=dtype)
    ops.branch_norm_add(branch.to(DEV), w.to(DEV), s.to(DEV), h2, eps, next_weight=w2.to(DEV), out=out, next_eps=eps2)
    assert torch.equal(h1, h2)
    assert _rel(out, want_x) < (1e-6 if dtype == torch.float32 else 1e-2)
    h3 = hidden.clone().to(DEV)
    ops.branch_norm_add(branch.to(DEV), w.to(DEV), None, h3, eps)
    assert _rel(h3, hidden.double() + plain.norm(branch.double(), w.double(), eps)) < 1e-6


def test_stream_add_and_scaled_embedding():
    from tokensprint_b200 import ops

    T, W, V = 5, 72, 30
    hidden, rows, vec = _randn(T, W, seed=80).float(), _randn(T, W, seed=81).float(), _randn(W, seed=82).float()
    h = hidden.clone().to(DEV)
    ops.stream_add(h, rows.to(DEV), vec.to(DEV))
    assert torch.allclose(h.cpu(), hidden + rows + vec, atol=1e-6)
    h = hidden.clone().to(DEV)
    ops.stream_add(h, None, vec.to(DEV))
    assert torch.allclose(h.cpu(), hidden + vec, atol=1e-6)
    for dtype in (torch.float32, torch.bfloat16):
        table = _randn(V, W, seed=83).to(dtype)
        ids = torch.tensor([3, 0, 29, 3, 7], dtype=torch.int32)
        out = torch.empty((T, W), device=DEV)
        ops.embed_gather(out, table.to(DEV), ids.to(DEV), 12.5)
        assert torch.equal(out.cpu(), table.float()[ids.long()] * 12.5)
