"""Each Porarax mechanism alone on the GPU against its plain function, on inputs made so that a fault shows: latent
attention over a window with one key that decides the result just inside and just outside the window, at page borders,
at the query's own position (both kernels, prompts' portions and single tokens, keys cut into ranges); the rotation of
neighbouring pairs with the unit-RMS norm; the output gate; the delta rule with a state that barely decays, so that
what was written hundreds of tokens back still decides the output, across steps, with a slot used again; routing by a
softmax restricted to the picked logits, with a bias and exact ties; the clamped experts with both clamps at work.
"""
import numpy as np
import pytest
import torch

from tinyllama_c_b200 import ops
from plain import porarax_plain as plain

pytestmark = pytest.mark.gpu
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def dev(a, dtype=torch.float32):
    return torch.tensor(np.asarray(a), dtype=dtype, device="cuda")


def draw(g, shape, scale, dtype):
    x = g.standard_normal(shape) * scale
    return plain.bf16_round(x) if dtype == "bfloat16" else x.astype(np.float32).astype(np.float64)


class _Step:
    pass


def _step_for(positions, slot=1):
    T = len(positions)
    step = _Step()
    step.n_seqs, step.n_rows, step.max_context = 1, T, int(max(positions)) + 1
    step.positions = dev(positions, torch.int32)
    step.row_seq = torch.zeros(T, dtype=torch.int32, device="cuda")
    step.cu_seqlens = dev([0, T], torch.int32)
    step.slots = dev([slot], torch.int32)
    step.start_pos = dev([positions[0]], torch.int32)
    return step


def _attend(qa, rows, scale, positions, H, R, window, dtype, tc, key_ranges=0):
    """ops.latent_attention (no sink, no rotated part) for one sequence whose pages lie scattered in the pool; pages
    wholly behind the window of the first query hold rubbish, as pages do that the cache gave back."""
    n_keys = rows.shape[0]
    n_pages = (n_keys + 63) // 64
    pool = 2 * n_pages + 3
    table = np.zeros((2, pool), dtype=np.int32)
    table[1, :n_pages] = [pool - 1 - 2 * i for i in range(n_pages)]
    pages = np.full((pool, 64, R), 7.0)
    first_kept = max(0, positions[0] + 1 - window) // 64
    for j in range(n_keys):
        pages[table[1, j // 64], j % 64] = rows[j] if j // 64 >= first_kept else 1e4
    T = len(positions)
    out = torch.empty((T, H * R), dtype=DT[dtype], device="cuda")
    try:
        ops.latent_attention_tc(tc)
        ops.latent_attention(dev(qa.reshape(T, -1), DT[dtype]), dev(pages, DT[dtype]), None, dev(table, torch.int32), _step_for(positions),
                             out, H, R, 0, scale, key_ranges, window=window)
    finally:
        ops.latent_attention_tc(True)
    torch.cuda.synchronize()
    return out.float().cpu().numpy().reshape(T, H, R)


def _attend_plain(q, rows, scale, p, window):
    """q [H, R]: softmax over keys max(0, p - window + 1) .. p of q . row, times the rows."""
    lo = max(0, p - window + 1)
    s = (rows[lo:p + 1] @ q.T) * scale                     # [keys, H]
    e = np.exp(s - s.max(0, keepdims=True))
    return (e / e.sum(0, keepdims=True)).T @ rows[lo:p + 1]


@pytest.mark.parametrize("H,R", [(3, 32), (2, 160), (5, 24)])
@pytest.mark.parametrize("kernel", ["warp32", "warp16", "tc", "tc3"])
@pytest.mark.parametrize("window", [1, 5, 64, 130, 1000])
def test_one_key_decides_just_inside_and_just_outside_the_window(kernel, H, R, window):
    """300 cached rows of small random values; one of them, `hot`, lines up with head 1's query and scores far above the
    rest.  Head 1's output is that row wherever the key is inside the query's window and the average of the visible rows
    where it is one step outside, beyond the query, or far behind."""
    dtype = "float32" if kernel == "warp32" else "bfloat16"
    tc, ranges = kernel.startswith("tc"), int(kernel[2:] or 1) if kernel.startswith("tc") else 0
    if tc and R % 16:
        pytest.skip("the tensor-core kernel takes latents that are multiples of 16")
    g = np.random.default_rng(11)
    n, scale = 300, 0.5
    for hot in (0, 63, 64, 150, 191, 192, 299):
        rows = draw(g, (n, R), 0.1, dtype)
        rows[hot] = draw(g, (R,), 1.0, dtype)
        cases = [[hot], [min(hot + window - 1, n - 1)], [min(hot + window, n - 1)], [max(hot - 1, 0)], [n - 1],
                 list(range(max(0, min(hot + window - 8, n - 16)), max(0, min(hot + window - 8, n - 16)) + 16))]
        for positions in cases:
            T = len(positions)
            qa = draw(g, (T, H, R), 0.1, dtype)
            hotq = rows[hot] * 6.0 * 48.0 / R
            qa[:, 1] = plain.bf16_round(hotq) if dtype == "bfloat16" else hotq
            got = _attend(qa, rows, scale, positions, H, R, window, dtype, tc, ranges)
            for i, p in enumerate(positions):
                want = _attend_plain(qa[i], rows, scale, p, window)
                err = np.abs(got[i] - want).max()
                assert err <= (3e-5 if dtype == "float32" else 1.5e-2) * max(np.abs(want).max(), 0.1), \
                    f"{kernel} window {window}: hot key {hot}, query at {p}: error {err:.3e}"
                if 0 <= p - hot < window and window > 1:          # the test's point: the hot key carries head 1
                    assert np.abs(want[1] - rows[hot]).max() < 0.35 * np.abs(rows[hot]).max()


@pytest.mark.parametrize("interleaved", [True, False])
@pytest.mark.parametrize("dim,stride,rot", [(16, 16, 16), (20, 20, 6), (12, 20, 0), (64, 64, 32), (200, 256, 100)])
def test_rotation_of_pairs_and_unit_rms(dim, stride, rot, interleaved):
    g = np.random.default_rng(3)
    T, H, KV, eps = 9, 3, 2, 1e-5
    positions = [0, 1, 2, 63, 64, 65, 1000, 4097, 7]
    lead = 5
    x = g.standard_normal((T, lead + (H + KV) * stride + 3)).astype(np.float32)
    freq = (37.0 ** (-2.0 * np.arange(rot // 2) / max(rot, 1))).astype(np.float32)
    for norm_eps in (eps, None):
        buf = dev(x)
        ops.qk_rotate_norm(buf, lead, lead + H * stride, H, KV, stride, dim, dev(freq), interleaved, norm_eps, dev(positions, torch.int32))
        got = buf.cpu().numpy().astype(np.float64)
        want = x.astype(np.float64).copy()
        ang = (np.asarray(positions, dtype=np.float32)[:, None] * freq[None, :]).astype(np.float64)
        for u in range(H + KV):
            head = want[:, lead + u * stride: lead + u * stride + dim]          # a view
            ia = np.arange(rot // 2) * 2 if interleaved else np.arange(rot // 2)
            ib = ia + 1 if interleaved else ia + rot // 2
            a, b = head[:, ia].copy(), head[:, ib].copy()
            head[:, ia] = a * np.cos(ang) - b * np.sin(ang)
            head[:, ib] = b * np.cos(ang) + a * np.sin(ang)
            if norm_eps is not None:
                head[:] = plain.unit_rms(head, norm_eps)
        assert np.abs(got - want).max() <= 2e-5 * 4.0, f"norm {norm_eps}: {np.abs(got - want).max():.3e}"
        # what lies between and behind the heads in use is untouched
        assert np.array_equal(got[:, :lead], x[:, :lead].astype(np.float64)) and np.array_equal(got[:, -3:], x[:, -3:].astype(np.float64))


@pytest.mark.parametrize("pad", [9, 12])            # (12: rows of the gate on 16-byte boundaries, four elements a thread)
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_output_gate(dtype, pad):
    g = np.random.default_rng(4)
    T, n = 7, 52
    x, gate = draw(g, (T, n), 1.0, dtype), g.standard_normal((T, n + pad)).astype(np.float32) * 3.0
    for kind, fn in (("sigmoid", plain.sigmoid), ("silu", plain.silu)):
        buf, gd = dev(x, DT[dtype]), dev(gate)
        ops.gate_mul(buf, gd[:, 4:4 + n], kind)
        want = x * fn(gate[:, 4:4 + n].astype(np.float64))
        assert np.abs(buf.float().cpu().numpy() - want).max() <= (1e-5 if dtype == "float32" else 1e-2) * np.abs(want).max()


def _delta_plain(q, k, v, beta, decay, H, G, dk, dv):
    T = q.shape[0]
    S = np.zeros((H, dk, dv))
    o = np.zeros((T, H, dv))
    for t in range(T):
        for h in range(H):
            kk, qq = k[t, h // (H // G)], q[t, h // (H // G)]
            S[h] *= decay[t, h]
            u = beta[t, h] * (v[t, h] - S[h].T @ kk)
            S[h] += np.outer(kk, u)
            o[t, h] = S[h].T @ qq
    return o


@pytest.mark.parametrize("split", [0, 8, 16])
@pytest.mark.parametrize("H,G,dk,dv", [(2, 1, 8, 8), (4, 2, 40, 12), (2, 2, 64, 64), (3, 3, 100, 33), (2, 1, 256, 16), (1, 1, 130, 70)])
def test_delta_rule_keeps_what_was_written_hundreds_of_tokens_back(H, G, dk, dv, split, request):
    """Two sequences in one step, then continued in portions and single tokens; decays within 1e-3 of one, and a value
    written at token 3 with a key that later queries repeat: the read-out hundreds of tokens later is mostly that value,
    so a state that is lost, reset, scaled twice or mixed up between sequences, heads or slots shows.  The slots held
    rubbish before (a sequence at position 0 starts from zero whatever its slot holds), and slot 0 is then used again by
    a third sequence."""
    ops.delta_rule_split(split)                     # threads that share a column group's rows: both shapes of the kernel
    request.addfinalizer(lambda: ops.delta_rule_split(0))
    g = np.random.default_rng(5)
    lens, portions = [330, 97], [[203, 1, 1, 61, 64], [90, 1, 1, 3, 2]]
    n_slots = 3
    state = torch.full((n_slots, H, dk, dv), 3.0, device="cuda")

    def make(T, seed):
        r = np.random.default_rng(seed)
        q, k = r.standard_normal((T, G, dk)), r.standard_normal((T, G, dk))
        unit = k[3] / np.sqrt((k[3] * k[3]).sum(-1, keepdims=True))
        for t in range(T):                                            # no other token writes along token 3's key
            if t != 3:
                k[t] -= (k[t] * unit).sum(-1, keepdims=True) * unit
        q[5:] = 0.15 * q[5:] + k[3][None] * 2.0                       # later queries ask for token 3's key
        v = r.standard_normal((T, H, dv)) * 0.1
        v[3] = r.standard_normal((H, dv)) * 3.0
        beta = plain.sigmoid(r.standard_normal((T, H)))
        beta[3] = 0.97
        decay = 1.0 - 1e-3 * r.random((T, H))
        f = lambda a: a.astype(np.float32).astype(np.float64)
        return [f(a) for a in (q, k, v, beta, decay)]

    def run(seqs, slots, cuts):
        """seqs: per sequence its five arrays; cuts: per sequence the portions; returns the outputs per sequence."""
        outs = [[] for _ in seqs]
        at = [0] * len(seqs)
        for s in range(max(len(c) for c in cuts)):
            live = [i for i in range(len(seqs)) if s < len(cuts[i])]
            counts = [cuts[i][s] for i in live]
            T = sum(counts)
            qkv = np.zeros((T, 2 * G * dk + H * dv + 2), dtype=np.float32)
            proj_b = np.zeros((T, H + 1), dtype=np.float32)
            decay = np.zeros((T, H), dtype=np.float32)
            o = 0
            for i, n in zip(live, counts):
                q, k, v, beta, dc = [a[at[i]:at[i] + n] for a in seqs[i]]
                qkv[o:o + n, 1:1 + G * dk] = q.reshape(n, -1)
                qkv[o:o + n, 1 + G * dk:1 + 2 * G * dk] = k.reshape(n, -1)
                qkv[o:o + n, 1 + 2 * G * dk:1 + 2 * G * dk + H * dv] = v.reshape(n, -1)
                proj_b[o:o + n, 1:] = np.log(beta / (1.0 - beta))
                decay[o:o + n] = dc
                o += n
            step = _Step()
            step.n_seqs, step.n_rows = len(live), T
            step.cu_seqlens = dev(np.concatenate([[0], np.cumsum(counts)]), torch.int32)
            step.slots = dev([slots[i] for i in live], torch.int32)
            step.start_pos = dev([at[i] for i in live], torch.int32)
            qd, bd = dev(qkv), torch.empty((T, H), device="cuda")
            ops.delta_prepare(qd, 1, 1 + G * dk, G, dk, 1e-6, dk ** -0.5, dev(proj_b), 1, H, bd)
            y = torch.empty((T, H * dv), device="cuda")
            ops.delta_rule(qd, 1, 1 + G * dk, 1 + 2 * G * dk, bd, dev(decay), state, step, y, H, G, dk, dv)
            torch.cuda.synchronize()
            y = y.cpu().numpy().astype(np.float64)
            o = 0
            for i, n in zip(live, counts):
                outs[i].append(y[o:o + n])
                at[i] += n
                o += n
        return [np.concatenate(x).reshape(-1, H, dv) for x in outs]

    def want_of(seq):
        q, k, v, beta, decay = seq
        qn = q / np.sqrt((q * q).sum(-1, keepdims=True) + 1e-6) * dk ** -0.5
        kn = k / np.sqrt((k * k).sum(-1, keepdims=True) + 1e-6)
        return _delta_plain(qn, kn, v, beta, decay, H, G, dk, dv)

    seqs = [make(n, 20 + i) for i, n in enumerate(lens)]
    got = run(seqs, [2, 0], portions)
    for i, seq in enumerate(seqs):
        want = want_of(seq)
        err = np.abs(got[i] - want).max()
        assert err <= 2e-5 * np.abs(want).max(), f"sequence {i}: error {err:.3e} of {np.abs(want).max():.3e}"
        # the test's point: far from token 3 the read-out is still mostly its value
        far = want[-1] / (dk ** -0.5)
        assert np.abs(far - seq[2][3]).max() < 0.5 * np.abs(seq[2][3]).max()
    third = make(40, 33)
    got3 = run([third], [0], [[1, 1, 30, 8]])[0]
    want3 = want_of(third)
    assert np.abs(got3 - want3).max() <= 2e-5 * np.abs(want3).max(), "a slot used again"


def test_routing_by_softmax_over_the_chosen_with_exact_ties():
    g = np.random.default_rng(6)
    for E, top in ((8, 2), (5, 5), (1, 1), (70, 6), (33, 1)):
        T = 50
        z = g.standard_normal((T, E + 2)).astype(np.float32)
        z[:10, :E] = np.round(z[:10, :E])                   # exact ties: the lowest index wins
        z[10, :E] = 0.0
        ids, wts, order, offsets, tile_off, _ = ops.moe_route(dev(z), E, top, 32, "softmax")
        torch.cuda.synchronize()
        ids, wts = ids.cpu().numpy().reshape(T, top), wts.cpu().numpy().reshape(T, top)
        for t in range(T):
            want_ids, want_w = plain.route(z[t, :E].astype(np.float64), top)
            assert list(ids[t]) == want_ids, f"E={E} top={top} token {t}"
            assert np.abs(wts[t] - want_w).max() <= 1e-6
            assert abs(wts[t].sum() - 1.0) <= 1e-5
        order, offsets = order.cpu().numpy(), offsets.cpu().numpy()
        flat = ids.reshape(-1)
        assert sorted(order.tolist()) == list(range(T * top))
        for e in range(E):
            assert all(flat[i] == e for i in order[offsets[e]:offsets[e + 1]])


@pytest.mark.parametrize("dtype,D,F", [("float32", 44, 20), ("float32", 64, 24), ("bfloat16", 64, 24), ("bfloat16", 44, 12), ("bfloat16", 128, 72)])
def test_clamped_experts_with_the_weight_on_their_output(dtype, D, F):
    """Inputs and weights large enough that the cut of the gate and both bounds of the up projection are at work in a
    good share of the elements; the CUDA-core products (32-bit, or rows that are not 16-byte aligned) and the tensor-core
    ones."""
    g = np.random.default_rng(8)
    E, top, T, limit = 6, 3, 75, 0.8
    W = {}
    for e in range(E):
        W[f"m.e{e}.gate"], W[f"m.e{e}.up"] = draw(g, (F, D), 0.3, dtype), draw(g, (F, D), 0.3, dtype)
        W[f"m.e{e}.down"] = draw(g, (D, F), 0.3, dtype)
    x = draw(g, (T, D), 1.0, dtype)
    z = g.standard_normal((T, E)).astype(np.float32)
    routing = ops.moe_route(dev(z), E, top, 32, "softmax")
    wgu = dev(np.stack([np.concatenate([W[f"m.e{e}.gate"], W[f"m.e{e}.up"]]) for e in range(E)]), DT[dtype])
    wd = dev(np.stack([W[f"m.e{e}.down"] for e in range(E)]), DT[dtype])
    act = torch.empty((T * top, F), dtype=DT[dtype], device="cuda")
    y = torch.empty((T, top, D), device="cuda")
    ops.moe_experts(dev(x, DT[dtype]), wgu, wd, routing, top, act, y, "swish_clamped", "output", limit, plain.SWISH_ALPHA)
    torch.cuda.synchronize()
    got = y.cpu().numpy().astype(np.float64)
    clipped = 0
    for t in range(T):
        ids, w = plain.route(z[t].astype(np.float64), top)
        for k, (e, wk) in enumerate(zip(ids, w)):
            want = wk * plain.expert(x[t], W, "m.", e, limit)
            tol = 2e-5 if dtype == "float32" else 2e-2
            assert np.abs(got[t, k] - want).max() <= tol * max(np.abs(want).max(), 0.5), f"token {t} choice {k}"
            clipped += int((W[f"m.e{e}.gate"] @ x[t] > limit).sum() + (np.abs(W[f"m.e{e}.up"] @ x[t]) > limit).sum())
    assert clipped > T * top * F // 4
