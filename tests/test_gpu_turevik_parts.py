"""Each Turevik mechanism alone on the GPU against its plain function: the norm with token shift and its kept row, the
output norm with its sum of terms, the GELU gate, minGRU (row by row and in chunks, with a slowly decaying state), the
product per head, latent attention as a mixer (own rows, and another entry's rows), its two kernels on inputs made so
that one key far back, at a page's border, at the query's own position or just beyond it decides the result, the sink,
routing (ties, every expert's list) and the experts.
"""
import numpy as np
import pytest
import torch

from tinyllama_c_b200 import ops
from tinyllama_c_b200.cache import Cache
from tinyllama_c_b200.engine.step import StepEntry, pack
from tinyllama_c_b200.parts.base import ChunkRequest, PartSpec
from plain import turevik_plain as plain

pytestmark = pytest.mark.gpu
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
TOL = {"float32": 2e-5, "bfloat16": 2e-2}
LENS = [1, 200, 70, 5]
DECODED = 6


def rnd_of(dtype):
    return plain.bf16_round if dtype == "bfloat16" else plain._same


def dev(a, dtype=torch.float32):
    return torch.tensor(np.asarray(a), dtype=dtype, device="cuda")


def draw(g, shape, scale, dtype):
    x = g.standard_normal(shape) * scale
    return plain.bf16_round(x) if dtype == "bfloat16" else x.astype(np.float32).astype(np.float64)


def run_steps(forward, requests, rows, dtype, in_dtype, chunk_requests=(), lens=LENS, kv_requests=None):
    """Feeds the sequences `rows` (one array [len + DECODED, width] each) through forward(x, step, views) -> [T, out]:
    all prompts in one step, then one token each.  `views`: the layer caches of entries 0 (and 1, which reads entry 0's
    keys where kv_requests gives it requests of its own)."""
    reqs = {0: requests}
    if kv_requests is not None:
        reqs[1] = kv_requests
    cache = Cache(reqs, max_tokens=64 * 8, max_seqs=len(lens), dtype=DT[dtype], device="cuda")
    slots = [cache.acquire() for _ in lens]
    got, done = [[] for _ in lens], [0] * len(lens)
    chunk_rows = [q.rows for q in chunk_requests]
    chunk_from = {q.rows: q.from_rows for q in chunk_requests if q.from_rows is not None}
    for s in range(1 + DECODED):
        counts = lens if s == 0 else [1] * len(lens)
        entries = [StepEntry(slot, [0] * n, ()) for slot, n in zip(slots, counts)]
        starts = [cache.reserve(e.slot, len(e.tokens)) for e in entries]
        step, _, _ = pack(entries, starts, 1, "cuda", chunk_rows, chunk_from)
        cache.upload_tables()
        x = np.concatenate([rows[b][done[b]:done[b] + n] for b, n in enumerate(counts)])
        views = [cache.layer_view(0)] + ([cache.layer_view(1, True, 0)] if kv_requests is not None else [])
        out = forward(dev(x, in_dtype), step, views)
        torch.cuda.synchronize()
        ops.check_errors()
        out = out.float().cpu().numpy()
        o = 0
        for b, n in enumerate(counts):
            got[b].append(out[o:o + n])
            o += n
            done[b] += n
            cache.commit(slots[b], n)
    for slot in slots:
        cache.release(slot)
    cache.check()
    return [np.concatenate(g) for g in got]


def compare(got, want, dtype, what, tol=None):
    for b, (g, w) in enumerate(zip(got, want)):
        err = np.abs(g - w).max()
        assert err <= (tol or TOL[dtype]) * np.abs(w).max(), f"{what}, sequence {b}: error {err:.3e} of {np.abs(w).max():.3e}"


# ---- norms, gate ------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", list(DT))
@pytest.mark.parametrize("width", [44, 256])
def test_norm_with_token_shift(dtype, width):
    g = np.random.default_rng(1)
    w, mu = g.standard_normal(width) * 0.1, g.random(width)
    part = PartSpec("norm", "rmsnorm_shift", dict(width=width, eps=1e-5, weight_name="w", mix_name="mu", offset=1.0)).build()
    part.bind({"w": torch.tensor(w, dtype=torch.float32), "mu": torch.tensor(mu, dtype=torch.float32)}, DT[dtype], "cuda")
    rows = [g.standard_normal((n + DECODED, width)) * 3.0 for n in LENS]

    def forward(x, step, views):
        out = torch.empty(x.shape, dtype=DT[dtype], device="cuda")
        return part.forward_step(x, out, step, views[0])
    got = run_steps(forward, part.cache_requests(), rows, dtype, torch.float32)
    f32 = lambda a: np.asarray(a, dtype=np.float32).astype(np.float64)
    want = [plain.token_shift(plain.offset_norm(f32(r), f32(w), 1e-5), f32(mu)) for r in rows]
    compare(got, want, dtype, "norm with token shift")


def test_output_norm_adds_terms_in_order():
    g = np.random.default_rng(2)
    T, n, D = 37, 3, 52
    parts, extra, gate = g.standard_normal((T, n, D)), g.standard_normal((T, D)), g.standard_normal((T, 4))
    res, w = g.standard_normal((T, D)), 1.0 + g.standard_normal(D) * 0.1
    y = parts.sum(axis=1) + plain.sigmoid(gate[:, 2:3]) * extra
    r = dev(res)
    ops.rmsnorm_add(dev(parts), dev(w), 1e-6, r, dev(extra), dev(gate)[:, 2], gate_sigmoid=True)
    want = res + plain.plain_norm(y, w, 1e-6)
    assert np.abs(r.cpu().numpy() - want).max() <= 1e-5 * np.abs(want).max()
    r = dev(res)
    ops.rmsnorm_add(dev(parts[:, 0]), None, 0.0, r, accumulate=False)            # one term, no norm, overwrite
    assert np.abs(r.cpu().numpy() - parts[:, 0]).max() <= 1e-6


@pytest.mark.parametrize("act", ["silu", "gelu_tanh"])
def test_gated_activation(act):
    g = np.random.default_rng(3)
    gu = g.standard_normal((19, 2 * 24)) * 3.0
    out = torch.empty((19, 24), dtype=torch.float32, device="cuda")
    ops.glu(dev(gu), out, act)
    f = plain.gelu_tanh if act == "gelu_tanh" else plain.silu
    want = f(gu[:, :24]) * gu[:, 24:]
    assert np.abs(out.cpu().numpy() - want).max() <= 2e-6 * np.abs(want).max()


@pytest.mark.parametrize("act", ["silu", "gelu_tanh"])
@pytest.mark.parametrize("dtype,D,F", [("bfloat16", 256, 2048), ("bfloat16", 64, 40), ("bfloat16", 44, 28), ("float32", 64, 40)])
def test_gated_feed_forward_with_either_activation(act, dtype, D, F):
    """The dense feed-forward part with its activation in the product's epilogue (bfloat16, widths that are multiples
    of 8: the kernels for 1..32, 17..128 and more rows) or as a kernel of its own."""
    g = np.random.default_rng(12)
    W = {"f.gate": draw(g, (F, D), 0.1, dtype), "f.up": draw(g, (F, D), 0.1, dtype), "f.down": draw(g, (D, F), 0.1, dtype)}
    part = PartSpec("feed_forward", "swiglu", dict(hidden=D, intermediate=F, prefix="f.", act=act,
                                                   names=dict(gate="gate", up="up", down="down"))).build()
    part.bind({k: torch.tensor(v, dtype=DT[dtype]) for k, v in W.items()}, DT[dtype], "cuda")
    f = plain.gelu_tanh if act == "gelu_tanh" else plain.silu
    for T in (1, 20, 40, 100, 300):
        x = draw(g, (T, D), 2.0, dtype)
        out = torch.zeros((T, D), dtype=torch.float32, device="cuda")
        part.forward(dev(x, DT[dtype]), out, accumulate=False)
        want = plain.gated_ff(x, W, "f.", f, rnd_of(dtype))
        err = np.abs(out.cpu().numpy() - want).max()
        assert err <= (3e-5 if dtype == "float32" else 2e-2) * np.abs(want).max(), f"{act} {T} rows: error {err:.3e}"


@pytest.mark.parametrize("dtype,T,K,pad,N", [("float32", 45, 20, 5, 37), ("bfloat16", 45, 20, 5, 37), ("bfloat16", 1, 24, 8, 37),
                                             ("bfloat16", 100, 72, 8, 70), ("bfloat16", 33, 16, 0, 64)])
def test_product_per_head(dtype, T, K, pad, N):
    """Heads that start inside wider rows; with 16-byte aligned bfloat16 rows the tensor-core kernel, else the CUDA cores."""
    g = np.random.default_rng(4)
    H = 3
    a, w = draw(g, (T, H, K + pad), 1.0, dtype), draw(g, (H, N, K), 1.0, dtype)
    out = torch.zeros((T, H * (N + 2)), dtype=torch.float32, device="cuda")
    ops.linear_heads(dev(a.reshape(T, -1), DT[dtype]), K + pad, dev(w, DT[dtype]), out, N + 2)
    want = np.einsum("thk,hnk->thn", a[:, :, :K], w)
    got = out.cpu().numpy().reshape(T, H, N + 2)
    assert np.abs(got[:, :, :N] - want).max() <= 1e-5 * np.abs(want).max()
    assert np.abs(got[:, :, N:]).max() == 0.0


# ---- minGRU ------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", list(DT))
@pytest.mark.parametrize("slow", [False, True])
def test_mingru_alone(dtype, slow):
    """slow: the gate's bias keeps z near 0.003, so the state of hundreds of tokens back still decides the output."""
    g = np.random.default_rng(5)
    D, Wd = 40, 72
    names = dict(z="z", z_bias="zb", x="x", x_bias="xb", g="g", o="o")
    W = {"z": draw(g, (Wd, D), 0.2, dtype), "x": draw(g, (Wd, D), 0.3, dtype), "g": draw(g, (Wd, D), 0.3, dtype),
         "o": draw(g, (D, Wd), 0.2, dtype), "zb": draw(g, (Wd,), 0.5, dtype) - (6.0 if slow else 0.0), "xb": draw(g, (Wd,), 0.5, dtype)}
    part = PartSpec("mixer", "mingru", dict(hidden=D, width=Wd, names=names)).build()
    part.bind({k: torch.tensor(v, dtype=DT[dtype] if v.ndim == 2 else torch.float32) for k, v in W.items()}, DT[dtype], "cuda")
    rows = [draw(g, (n + DECODED, D), 1.0, dtype) for n in LENS]

    def forward(x, step, views):
        out = torch.zeros((x.shape[0], D), dtype=torch.float32, device="cuda")
        part.forward(x, step, views[0], out, accumulate=False)
        return out
    got = run_steps(forward, part.cache_requests(), rows, dtype, DT[dtype], part.step_requests())
    Wp = {"m." + dict(zb="z.b", xb="x.b").get(k, k): v for k, v in W.items()}
    want = [plain.mingru(r, Wp, "m.", rnd=rnd_of(dtype))[0] for r in rows]
    compare(got, want, dtype, "minGRU")


# ---- latent attention ------------------------------------------------------------------------------------------------
def latent_parts(g, dtype, D, H, dn, r, dv, R, dims, H2, dn2, dv2):
    m1 = dict(heads=H, dim=dn, rot_dim=r, vdim=dv, kv_rank=R, scale=0.3, rot=dict(base=1000.0, dims=dims))
    m2 = dict(m1, heads=H2, dim=dn2, vdim=dv2, scale=0.2)
    W = {}
    for p, m, own in (("a.", m1, True), ("b.", m2, False)):
        W[p + "q"] = draw(g, (m["heads"] * (m["dim"] + r), D), 0.3, dtype)
        W[p + "uk"] = draw(g, (m["heads"] * m["dim"], R), 0.3, dtype)
        W[p + "uv"] = draw(g, (m["heads"] * m["vdim"], R), 0.3, dtype)
        W[p + "o"] = draw(g, (D, m["heads"] * m["vdim"]), 0.3, dtype)
        W[p + "sink"] = draw(g, (m["heads"],), 1.0, dtype)
        if own:
            W[p + "dkv"] = draw(g, (R + r, D), 0.3, dtype)
            W[p + "dkv.norm"] = 1.0 + draw(g, (R,), 0.1, dtype)
    parts = []
    for p, m, own in (("a.", m1, True), ("b.", m2, False)):
        names = {k: p + v for k, v in dict(q="q", dkv="dkv", dkv_norm="dkv.norm", uk="uk", uv="uv", sink="sink", o="o").items()}
        part = PartSpec("mixer", "latent_attention", dict(
            hidden=D, n_heads=m["heads"], head_dim=m["dim"], rot_dim=r, v_dim=m["vdim"], kv_rank=R, scale=m["scale"], eps=1e-5,
            position=PartSpec("position", "rope_interleaved", dict(head_dim=r, theta=1000.0, rope_dim=dims)), names=names,
            own_latent=own)).build()
        part.bind({k: torch.tensor(v, dtype=DT[dtype] if v.ndim == 2 else torch.float32) for k, v in W.items()}, DT[dtype], "cuda")
        parts.append(part)
    return W, m1, m2, parts


@pytest.mark.parametrize("dtype", list(DT))
@pytest.mark.parametrize("sizes", [(3, 8, 16, 24, 32, 16, 2, 16, 8), (1, 12, 16, 12, 48, 8, 5, 4, 20), (4, 8, 8, 8, 48, 8, 2, 8, 8)])
def test_latent_attention_own_rows_and_another_entrys(dtype, sizes):
    """Entry 0 stores rows and attends; entry 1 has no down-projection and attends over entry 0's rows with its own
    queries, up-projections, head sizes and sink.  (48 + 8 = 56 columns: the warp kernel also in bfloat16.)"""
    H, dn, r, dv, R, dims, H2, dn2, dv2 = sizes
    g = np.random.default_rng(6)
    D = 40
    W, m1, m2, (own, borrower) = latent_parts(g, dtype, D, H, dn, r, dv, R, dims, H2, dn2, dv2)
    rows = [draw(g, (n + DECODED, D), 1.0, dtype) for n in LENS]

    def forward(x, step, views):
        out = torch.zeros((x.shape[0], 2 * D), dtype=torch.float32, device="cuda")
        a, b = torch.zeros((x.shape[0], D), dtype=torch.float32, device="cuda"), torch.zeros((x.shape[0], D), dtype=torch.float32, device="cuda")
        own.forward(x, step, views[0], a, accumulate=False)
        borrower.forward(x, step, views[1], b, accumulate=False)
        out[:, :D], out[:, D:] = a, b
        return out
    got = run_steps(forward, own.cache_requests(), rows, dtype, DT[dtype], kv_requests=[])
    rn = rnd_of(dtype)
    want = []
    for x in rows:
        pos = np.arange(len(x))
        c, kr = plain.latent_cache_rows(x, W, "a.", m1, 1e-5, pos, rn)
        want.append(np.concatenate([plain.latent_attention(x, W, "a.", m1, pos, c, kr, rn),
                                    plain.latent_attention(x, W, "b.", m2, pos, c, kr, rn)], axis=1))
    compare(got, want, dtype, "latent attention", tol=3e-5 if dtype == "float32" else 4e-2)


class _Step:
    pass


def _attend(qa, rows, sink, scale, positions, H, R, r, dtype, tc, key_ranges=0):
    """ops.latent_attention for one sequence whose pages lie scattered and out of order in the pool."""
    n_keys = rows.shape[0]
    n_pages = (n_keys + 63) // 64
    pool = 2 * n_pages + 3
    table = np.zeros((2, pool), dtype=np.int32)
    table[1, :n_pages] = [pool - 1 - 2 * i for i in range(n_pages)]              # slot 1; descending, every other page
    pages = np.full((pool, 64, R + r), 7.0)                                       # what other pages hold must not matter
    for j in range(n_keys):
        pages[table[1, j // 64], j % 64] = rows[j]
    T = len(positions)
    step = _Step()
    step.n_seqs, step.max_context = 1, int(max(positions)) + 1
    step.positions = dev(positions, torch.int32)
    step.row_seq = torch.zeros(T, dtype=torch.int32, device="cuda")
    step.cu_seqlens = dev([0, T], torch.int32)
    step.slots = dev([1], torch.int32)
    step.start_pos = dev([positions[0]], torch.int32)
    out = torch.empty((T, H * R), dtype=DT[dtype], device="cuda")
    try:
        ops.latent_attention_tc(tc)
        ops.latent_attention(dev(qa.reshape(T, -1), DT[dtype]), dev(pages, DT[dtype]), dev(sink), dev(table, torch.int32), step, out,
                             H, R, r, scale, key_ranges)
    finally:
        ops.latent_attention_tc(True)
    torch.cuda.synchronize()
    return out.float().cpu().numpy().reshape(T, H, R)


@pytest.mark.parametrize("sizes", [(3, 32, 16), (70, 16, 16), (2, 160, 32)])
@pytest.mark.parametrize("kernel", ["warp32", "warp16", "tc", "tc3", "tc5"])
def test_one_key_decides_far_back_at_page_borders_own_position_and_beyond(kernel, sizes):
    """300 cached rows of small random values; one of them, `hot`, lines up with head 1's query and scores far above the
    rest, so the output of head 1 is that row's latent wherever the key is visible and the plain average where it is
    not: keys at position 0, at both sides of the page borders, far back, at the query's own position and one beyond it
    (what a freed page or a later token left there).  Queries are consecutive rows of a prompt's portion, or a single
    decoded token."""
    dtype = "float32" if kernel == "warp32" else "bfloat16"
    tc, ranges = kernel.startswith("tc"), int(kernel[2:] or 1) if kernel.startswith("tc") else 0
    g = np.random.default_rng(7)
    (H, R, r), scale = sizes, 0.5          # (70 heads: two groups of 64 a row; a latent of 160: the wider accumulator)
    n = 300
    for hot in ((0, 63, 64, 127, 128, 255, 256, 290, 299) if H == 3 else (0, 64, 127, 299)):
        rows = draw(g, (n, R + r), 0.1, dtype)
        rows[hot] = draw(g, (R + r,), 1.0, dtype)
        sink = np.resize(np.array([0.0, -1.0, 0.5]), H)
        for positions in (list(range(284, 300)), [hot], [max(hot - 1, 0)], [299]):
            T = len(positions)
            qa = draw(g, (T, H, R + r), 0.1, dtype)
            qa[:, 1] = plain.bf16_round(rows[hot] * 6.0 * 48.0 / (R + r)) if dtype == "bfloat16" else rows[hot] * 6.0 * 48.0 / (R + r)
            got = _attend(qa, rows, sink, scale, positions, H, R, r, dtype, tc, ranges)
            for i, p in enumerate(positions):
                want = plain.attend_latent(qa[i], rows, sink, scale, p + 1)[:, :R]
                err = np.abs(got[i] - want).max()
                assert err <= (3e-5 if dtype == "float32" else 1.5e-2) * max(np.abs(want).max(), 0.1), \
                    f"{kernel}: hot key {hot}, query at {p}: error {err:.3e}"
                if hot <= p:                       # the test's point: the hot key carries head 1
                    assert np.abs(want[1] - rows[hot, :R]).max() < 0.35 * np.abs(rows[hot, :R]).max()


@pytest.mark.parametrize("kernel", ["warp", "tc", "tc4"])
def test_sink_takes_its_share(kernel):
    """A sink far above every score leaves almost nothing for the keys; one far below changes nothing."""
    tc, ranges = kernel.startswith("tc"), int(kernel[2:] or 1) if kernel.startswith("tc") else 0
    g = np.random.default_rng(8)
    H, R, r = 2, 16, 16
    rows, qa = draw(g, (130, R + r), 1.0, "bfloat16"), draw(g, (1, H, R + r), 0.3, "bfloat16")
    for sink in (np.array([9.0, -30.0]), np.array([-30.0, 9.0])):
        got = _attend(qa, rows, sink, 0.25, [129], H, R, r, "bfloat16", tc, ranges)[0]
        want = plain.attend_latent(qa[0], rows, sink, 0.25, 130)[:, :R]
        assert np.abs(got - want).max() <= 1.5e-2 * np.abs(want).max()
        big = int(np.argmax(sink))
        assert np.abs(want[big]).max() < 0.5 * np.abs(want[1 - big]).max()


# ---- experts ---------------------------------------------------------------------------------------------------------
def test_routing_ties_weights_and_every_experts_list():
    g = np.random.default_rng(9)
    T, E, top = 300, 7, 3
    logits = np.round(g.standard_normal((T, E + 2)) * 2.0) / 2.0                  # many exact ties
    ids, wts, order, offsets, tile_off, _ = ops.moe_route(dev(logits), E, top)
    torch.cuda.synchronize()
    ids, wts, order, offsets, tile_off = (t.cpu().numpy() for t in (ids, wts, order, offsets, tile_off))
    want = np.argsort(-logits[:, :E], axis=1, kind="stable")[:, :top]
    assert (ids.reshape(T, top) == want).all()
    assert np.abs(wts.reshape(T, top) - plain.sigmoid(np.take_along_axis(logits[:, :E], want, 1))).max() < 1e-6
    assert offsets[0] == 0 and offsets[E] == T * top and sorted(order.tolist()) == list(range(T * top))
    for e in range(E):
        mine = order[offsets[e]:offsets[e + 1]]
        assert (ids[mine] == e).all() and len(mine) == (ids == e).sum()
        assert tile_off[e + 1] - tile_off[e] == (len(mine) + 31) // 32


@pytest.mark.parametrize("dtype,E,top,shared,D,F", [("float32", 6, 2, 20, 44, 28), ("float32", 3, 1, None, 44, 28),
                                                    ("float32", 40, 4, 12, 44, 28), ("bfloat16", 5, 5, 20, 44, 28),
                                                    ("bfloat16", 1, 1, None, 44, 28), ("bfloat16", 5, 5, 24, 48, 40),
                                                    ("bfloat16", 3, 3, None, 136, 72), ("bfloat16", 2, 2, 16, 64, 48)])
def test_experts_alone(dtype, E, top, shared, D, F):
    """(Widths that are multiples of 8 in bfloat16: the tensor-core kernel; else the CUDA cores.)"""
    g = np.random.default_rng(10)
    mlp = dict(router=dict(experts=E, top=top), expert=dict(ff=F), shared=None if shared is None else dict(ff=shared))
    W = {"f.router": draw(g, (E, D), 0.5, dtype)}
    for e in range(E):
        W.update({f"f.e{e}.gate": draw(g, (F, D), 0.3, dtype), f"f.e{e}.up": draw(g, (F, D), 0.3, dtype),
                  f"f.e{e}.down": draw(g, (D, F), 0.3, dtype)})
    spec = None
    if shared is not None:
        W.update({"f.shared.gate": draw(g, (shared, D), 0.3, dtype), "f.shared.up": draw(g, (shared, D), 0.3, dtype),
                  "f.shared.down": draw(g, (D, shared), 0.3, dtype), "f.shared.sg": draw(g, (1, D), 0.3, dtype)})
        spec = PartSpec("feed_forward", "swiglu", dict(hidden=D, intermediate=shared, prefix="f.shared.",
                                                       names=dict(gate="gate", up="up", down="down")))
    part = PartSpec("feed_forward", "moe", dict(hidden=D, n_experts=E, top=top, expert_ff=F, router_name="f.router",
                                                expert_names={k: "f.e{e}." + k for k in ("gate", "up", "down")}, shared=spec,
                                                shared_gate_name=None if shared is None else "f.shared.sg")).build()
    part.bind({k: torch.tensor(v, dtype=DT[dtype]) for k, v in W.items()}, DT[dtype], "cuda")
    for T in (1, 3, 150, 333):          # (333 rows: tiles of 64 rows where every expert gets that many)
        x = draw(g, (T, D), 1.0, dtype)
        out = torch.zeros((T, D), dtype=torch.float32, device="cuda")
        part.forward(dev(x, DT[dtype]), out, accumulate=False)
        want = plain.moe_ff(x, W, "f.", mlp, rnd_of(dtype))
        err = np.abs(out.cpu().numpy() - want).max()
        assert err <= (3e-5 if dtype == "float32" else 3e-2) * np.abs(want).max(), f"{T} rows: error {err:.3e}"
        alone = torch.zeros((1, D), dtype=torch.float32, device="cuda")           # a row's result does not depend on the batch
        part.forward(dev(x[T - 1:T], DT[dtype]), alone, accumulate=False)
        assert np.abs(alone.cpu().numpy()[0] - out.cpu().numpy()[T - 1]).max() <= (1e-5 if dtype == "float32" else 5e-3) * np.abs(want).max()
