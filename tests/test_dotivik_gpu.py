"""Dotivik through the engine against the plain implementation of tests/plain/dotivik_plain.py.

Small configurations made here (none is anyone's model), random weights from a seed.  Covered: the
kernels of each mechanism alone (layer norm with two pending products, the stream input's packing, the
gated activation, rotation and append of score maps, the latent row, one small matrix per head, the
combination of the maps), attention kernels with keys made to stand out far back, just inside and just
outside a window, at the first positions and at page borders; whole prompts; prefill against
token-by-token decoding (through captured graphs); portions down to two tokens; mixed batches over a
tight pool whose freed pages are poisoned; slots used again; long decoding; sizes that are equal or 1;
generation through Engine and its scheduler; the command line; bin/trace_run.
"""
import copy
import gc
import json
import math

import pytest
import torch

import schedules as S
from conftest import TraceRun, random_tokens, row_rms_error
from plain import dotivik_plain as P

pytestmark = pytest.mark.gpu


def maps(heads, kv_heads, dim, vdim, rot, base=3000.0, scale=0.3, softcap=30.0, diff=0.5, window=None):
    m = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=scale, softcap=softcap, diff=diff,
             rot=dict(dims=rot, base=base))
    if window is not None:
        m["mask"] = dict(size=window)
    return m


def latent(heads, dim, rot_dim, vdim, rank, window, base=3000.0, scale=0.3):
    m = dict(heads=heads, dim=dim, rot_dim=rot_dim, vdim=vdim, kv_rank=rank, scale=scale, rot=dict(dims=rot_dim, base=base))
    if window is not None:
        m["mask"] = dict(size=window)
    return m


def layer(kind, mixer, ff=None):
    return dict(type=kind, mixer=mixer, mlp=None if ff is None else dict(kind="dense", ff=ff))


def model(vocab, width, layers, loop=None, eps=1e-5):
    cfg = dict(architecture="Dotivik", vocab=vocab, width=width, norm=dict(eps=eps), layers=layers)
    if loop is not None:
        cfg["loop"] = dict(start=loop[0], stop=loop[1], times=loop[2])
    return cfg


# A: every branch at once: both mixers inside and outside a run of layers that repeats three times, grouped
# KV heads, maps rotated on a part of their width, a layer without a feed-forward, windows shorter than the
# test sequences, widths that are multiples of 8 (tensor-core attention in bfloat16).
CFG_A = model(211, 96, [
    layer("latent_attention", latent(6, 24, 8, 40, 48, 37), ff=160),
    layer("attention", maps(6, 2, 32, 48, 8), ff=64),
    layer("latent_attention", latent(3, 16, 16, 16, 40, 21, base=100.0)),
    layer("attention", maps(4, 4, 16, 24, 16, base=100.0, scale=0.5, softcap=5.0, diff=0.2), ff=72)], loop=(1, 3, 3))
# B: values that the usual model makes different are equal or 1 here: one head, as many KV heads as heads,
# values as wide as a map, a window of one key, a latent as wide as a head, a run that repeats once, no
# cap on the scores, a width that no tensor-core product takes (not a multiple of 8).
CFG_B = model(97, 100, [
    layer("attention", maps(1, 1, 24, 24, 24, scale=1.0, softcap=None, diff=0.8), ff=40),
    layer("latent_attention", latent(1, 20, 2, 20, 20, 1, scale=1.0)),
    layer("latent_attention", latent(3, 12, 4, 12, 12, 9, scale=0.7), ff=50),
    layer("attention", maps(3, 3, 10, 10, 0, scale=0.7, diff=0.5, window=33))], loop=(0, 4, 1))
# C: sizes of a real model's order (maps 64 wide, values 128, a cache row of 128), many heads on one row,
# no repeated layers at all, a window longer than any test sequence.
CFG_C = model(300, 256, [
    layer("latent_attention", latent(20, 64, 32, 64, 96, 500, base=1e6, scale=0.1), ff=512),
    layer("attention", maps(8, 1, 64, 128, 32, base=1e6, scale=0.125, softcap=50.0, diff=0.6), ff=384)])
# D: the repeated run covers every layer and opens the model; widths beyond the tensor-core tiles (a cache row
# of 160, maps 136 wide): the CUDA-core attention serves bfloat16 too.
CFG_D = model(150, 128, [
    layer("latent_attention", latent(4, 32, 32, 48, 128, 90, scale=0.2), ff=256),
    layer("attention", maps(2, 1, 136, 40, 64, scale=0.1, softcap=8.0, diff=0.3), ff=128)], loop=(0, 2, 2))
CONFIGS = {"A": CFG_A, "B": CFG_B, "C": CFG_C, "D": CFG_D}
# A row's error: the root mean square of (got - plain) as a share of the row's root mean square.  float32:
# every row within rounding of another summation order (the sharp comparison: see the sensitivity test).
# bfloat16: the mean over rows is held tightly and the worst row loosely (the difference of two softmax maps,
# divided by its own root mean square, amplifies the rounding of q and k at rows where the maps nearly
# cancel); what is sharp in bfloat16 is every schedule against the WHOLE prompt in the same dtype.
BF16_MEAN, BF16_WORST = 0.03, 0.6
F32_ROW = 4e-5
BF16_CUT = 0.1


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    from mini_hisparse_b200 import write_random_model

    out = {}
    for name, cfg in CONFIGS.items():
        folder = tmp_path_factory.mktemp(f"dotivik{name}")
        write_random_model(cfg, 29, folder, dtype=torch.bfloat16, matrix_std=0.15)
        out[name] = (folder, *P.load_folder(folder))
    return out


def requests_for(cfg, lengths, seed=0):
    return {f"r{i}": random_tokens(cfg["vocab"], n, seed + i) for i, n in enumerate(lengths)}


def run_steps(folder, dtype, steps, page_size=16, max_requests=4, graphs=True, round_to=64):
    """Replay ``steps`` through the step function over a pool sized like the replay program's, with
    poison on freed pages; returns {request: logits of all its positions}."""
    from mini_hisparse_b200 import CacheConfig, CacheManager, load_model
    from mini_hisparse_b200.engine import ModelRunner, StepEntry

    model = load_model(folder, dtype=dtype)
    unit = max(round_to, page_size)
    pages = -(-S.peak_tokens(steps, unit) // page_size)
    cache = CacheManager(model.cache_needs, CacheConfig(num_pages=pages, page_size=page_size, max_requests=max_requests,
                                                        dtype=model.rt.dtype, debug_poison=True))
    runner = ModelRunner(model, cache, use_graphs=graphs)
    got = {}
    for entries, end in steps:
        for e in entries:
            if e["id"] not in cache.requests:
                cache.open(e["id"])
        logits = runner.step([StepEntry(e["id"], e["tokens"], e["want"]) for e in entries]).cpu()
        runner.check_status()
        row = 0
        for e in entries:
            got.setdefault(e["id"], []).append(logits[row: row + len(e["want"])].clone())
            row += len(e["want"])
        for rid in end:
            cache.close(rid)
    cache.assert_invariants()
    stats, pages = dict(runner.stats), cache.snapshot()
    del runner, model
    gc.collect()                 # captured graphs and pools go now, not inside a later runner's capture
    return {k: torch.cat(v) for k, v in got.items()}, stats, pages


def check_against_plain(got, refs, dtype):
    for rid, ref in refs.items():
        assert got[rid].shape == ref.shape
        err = (got[rid].double() - ref.double()).pow(2).mean(-1).sqrt() / ref.double().pow(2).mean(-1).sqrt()
        if dtype == "float32":
            assert float(err.max()) < F32_ROW, f"{rid}: row error {float(err.max()):.3g} at {int(err.argmax())}"
        else:
            assert float(err.mean()) < BF16_MEAN and float(err.max()) < BF16_WORST, \
                f"{rid}: mean row error {float(err.mean()):.3g}, worst {float(err.max()):.3g} at {int(err.argmax())}"


def dev_i(t):
    return torch.as_tensor(t).to(torch.int32).cuda()


class Parts:
    """A pending product as the kernels' wrappers take it."""

    def __init__(self, tensor, nsplit=1):
        self.tensor, self.nsplit = tensor, nsplit
        self.split_stride = tensor.stride(0) if nsplit > 1 else 0


# ---- the kernels of each mechanism alone --------------------------------------------------------------
@pytest.mark.parametrize("H", [100, 192, 1000])
def test_layer_norm_adds_two_pending_products(H):
    from mini_hisparse_b200.kernels import api as K

    g = torch.Generator().manual_seed(1)
    T = 7
    x = 3 * torch.randn(T, H, generator=g) + 2.0            # a mean that is not zero: it must be taken off
    d1, d2 = torch.randn(3, T, H, generator=g), torch.randn(T, H, generator=g)
    w = 1 + 0.1 * torch.randn(H, generator=g)
    total = x.double() + d1.double().sum(0) + d2.double()
    for out_dtype, tol in ((torch.float32, 3e-6), (torch.bfloat16, 1e-2)):
        xd, out = x.cuda().clone(), torch.empty(T, H, dtype=out_dtype, device="cuda")
        K.add_layernorm(xd, w.cuda(), 1e-5, out, delta=Parts(d1.cuda(), 3), delta2=Parts(d2.cuda()))
        torch.testing.assert_close(xd.cpu().double(), total, atol=3e-6, rtol=3e-6)        # the sum is written back
        torch.testing.assert_close(out.float().cpu().double(), P.layer_norm(total, w.double(), 1e-5), atol=tol, rtol=tol)
    # chosen rows only (the last norm before the head): the stream stays as it is
    rows = torch.tensor([5, 0, 5], dtype=torch.int32)
    xd, out = x.cuda().clone(), torch.empty(3, H, device="cuda")
    K.add_layernorm(xd, w.cuda(), 1e-5, out, delta=Parts(d2.cuda()), rows=rows.cuda())
    torch.testing.assert_close(xd.cpu(), x, atol=0, rtol=0)
    ref = P.layer_norm((x.double() + d2.double())[rows.long()], w.double(), 1e-5)
    torch.testing.assert_close(out.cpu().double(), ref, atol=3e-6, rtol=3e-6)
    # nothing pending
    K.add_layernorm(xd, w.cuda(), 1e-5, out[:2], rows=rows[:2].cuda())
    torch.testing.assert_close(out[:2].cpu().double(), P.layer_norm(x.double()[rows[:2].long()], w.double(), 1e-5),
                               atol=3e-6, rtol=3e-6)


def test_a_pair_of_pending_products_reaches_a_norm_that_adds_one():
    """A parallel block leaves two products pending; a norm whose kernel adds one (the RMS norm of another
    arrangement that may follow) settles the second into the stream first."""
    from mini_hisparse_b200.engine.engine import make_runtime
    from mini_hisparse_b200.parts.base import Product, StepContext, Workspace
    from mini_hisparse_b200.parts.registry import NORMS
    from mini_hisparse_b200.parts.spec import PartSpec

    g = torch.Generator().manual_seed(6)
    T, H = 5, 72
    x, a, f = (torch.randn(T, H, generator=g) for _ in range(3))
    parts = torch.randn(2, T, H, generator=g)
    w = 1 + 0.1 * torch.randn(H, generator=g)
    rt = make_runtime("cuda:0", "float32")
    ctx = StepContext(rt=rt, ws=Workspace(rt.device), T=T, segments=[], tokens=None, positions=None, tok_seg=None,
                      seg_slot=None, status=None)
    norm = NORMS.build(PartSpec.make("rmsnorm", width=H, eps=1e-5), rt=rt)
    norm.load({"weight": w.cuda()})
    xd = x.cuda().clone()
    pending = Product(a.cuda(), 1, also=Product(parts.cuda(), 2, also=Product(f.cuda())))
    out = norm.forward(xd, ctx, delta=pending)
    total = x.double() + a.double() + parts.double().sum(0) + f.double()
    torch.testing.assert_close(xd.cpu().double(), total, atol=3e-6, rtol=3e-6)
    torch.testing.assert_close(out.cpu().double(), P.unit_rms(total, 1e-5) * w.double(), atol=3e-6, rtol=3e-6)
    torch.testing.assert_close(pending.reduced().cpu().double(), total - x.double(), atol=3e-6, rtol=3e-6)


def test_stream_packing_and_gated_activation():
    from mini_hisparse_b200.kernels import api as K

    g = torch.Generator().manual_seed(2)
    T, W = 5, 36
    x, d1, d2 = torch.randn(T, W, generator=g), torch.randn(2, T, W, generator=g), torch.randn(T, W, generator=g)
    cat = torch.full((T, 2 * W), 7.0, device="cuda")
    xd = x.cuda().clone()
    K.stream_pack(xd, cat, W)                                 # the right half, the stream untouched
    K.stream_pack(xd, cat, 0, delta=Parts(d1.cuda(), 2), delta2=Parts(d2.cuda()), zero=True)
    assert float(xd.abs().max()) == 0.0
    torch.testing.assert_close(cat.cpu(), torch.cat((x + d1.sum(0) + d2, x), 1), atol=1e-6, rtol=1e-6)
    z = 2 * torch.randn(2, T, 2 * 24, generator=g)             # two parts; blocks of 8 gate values, then 8 up values
    for act, f in (("gelu_tanh", P.gelu_tanh), ("silu", lambda v: v * torch.sigmoid(v))):
        out = torch.empty(T, 24, device="cuda")
        K.glu_act(z.cuda(), out, act, nsplit=2, split_stride=T * 48, block=8)
        zs = z.double().sum(0).view(T, 3, 2, 8)
        torch.testing.assert_close(out.cpu().double(), (f(zs[:, :, 0]) * zs[:, :, 1]).reshape(T, 24), atol=2e-6, rtol=2e-6)


@pytest.mark.parametrize("T,H,Kd,N,off,pad", [(37, 3, 20, 70, 3, 6), (150, 5, 96, 128, 8, 16), (70, 2, 40, 24, 0, 0)])
def test_one_small_matrix_per_head_through_strided_views(T, H, Kd, N, off, pad):
    """x and out are runs of columns of wider rows.  In bfloat16, strides and offsets that are multiples of 8
    take the tensor-core kernel (K padded to 32 inside), the others the CUDA cores."""
    from mini_hisparse_b200.kernels import api as K

    g = torch.Generator().manual_seed(3)
    wide_in, wide_out = torch.randn(T, H, Kd + pad, generator=g), torch.zeros(T, H, N + 5)
    w = torch.randn(H, N, Kd, generator=g)
    for dtype, tol in ((torch.float32, 1e-5), (torch.bfloat16, 2e-2)):
        xi, wo = wide_in.to(dtype).cuda(), wide_out.to(dtype).cuda()
        K.head_linear(xi[:, :, off:off + Kd], w.to(dtype).cuda(), wo[:, :, :N])
        ref = torch.einsum("thk,hnk->thn", xi[:, :, off:off + Kd].double().cpu(), w.to(dtype).double())
        torch.testing.assert_close(wo[:, :, :N].double().cpu(), ref, atol=tol * float(ref.abs().max()), rtol=0)
        assert float(wo[:, :, N:].abs().max()) == 0.0         # nothing beyond the view
        if dtype == torch.bfloat16:                            # float32 out of bfloat16 operands
            wf = torch.zeros(T, H, N, device="cuda")
            K.head_linear(xi[:, :, off:off + Kd], w.to(dtype).cuda(), wf)
            torch.testing.assert_close(wf.double().cpu(), ref, atol=1e-5 * float(ref.abs().max()), rtol=0)


def plain_maps_attention(q, k, v, qpos, scale, cap, window=None):
    """q [R, H, M, d] at positions qpos against keys k [L, G, M, d] and values v [L, G, dv] at positions
    0..L-1: [R, H, M, dv], every map a softmax of its own over the same values."""
    R, H, M, _ = q.shape
    G = k.shape[1]
    kpos = torch.arange(k.shape[0])
    diff = qpos[:, None] - kpos[None, :]
    seen = diff >= 0 if window is None else (diff >= 0) & (diff < window)
    out = torch.zeros(R, H, M, v.shape[2], dtype=torch.float64)
    for h in range(H):
        for m in range(M):
            s = (q[:, h, m] @ k[:, h // (H // G), m].T) * scale
            if cap:
                s = cap * torch.tanh(s / cap)
            out[:, h, m] = torch.softmax(s.masked_fill(~seen, -math.inf), -1) @ v[:, h // (H // G)]
    return out


def attend(K, kernel, dtype, shape, segments, q_rows, pool, table, out_shape, out_dtype, **opts):
    """Plan the step's attention and run the chosen kernel family over it."""
    from mini_hisparse_b200.parts.attention import plan_attention

    T = sum(s.count for s in segments)
    plan = plan_attention(shape, segments, T, sm_count=148)
    n = plan.n_small + plan.n_big
    nq, dv = out_shape
    part_acc = torch.empty(max(1, plan.part_rows), nq, dv, device="cuda")
    part_ml = torch.empty(max(1, plan.part_rows), nq, 2, device="cuda")
    o = torch.zeros(T, nq, dv, dtype=out_dtype, device="cuda")
    tables = dev_i(table[None, :].repeat(len(segments), 1))
    positions = dev_i(torch.cat([torch.arange(s.start, s.start + s.count) for s in segments]))
    items = dev_i(torch.from_numpy(plan.items))
    tpr, tns = dev_i(torch.from_numpy(plan.tok_part_row)), dev_i(torch.from_numpy(plan.tok_nsplit))
    gate = {k: opts[k] for k in ("gate", "gate_nsplit", "gate_split_stride", "gate_per_head") if k in opts}
    if kernel in ("mma", "tc"):
        if plan.n_small:
            counters = torch.zeros(T * opts["nkv"] * opts.get("kparts", 1) * -(-(shape.q_heads // shape.kv_heads) // 16),
                                   dtype=torch.int32, device="cuda")
            if kernel == "tc":          # TMA-fed 16-row tiles
                status = torch.zeros(1, dtype=torch.int32, device="cuda")
                tc = {k: v for k, v in opts.items() if k not in ("dv", "kparts")}
                K.attention_tma_ext(q_rows, pool, o, part_acc, part_ml, items, plan.n_small, 16, positions, tables, tpr,
                                    **tc, tok_nsplit=tns, counters=counters, status=status)
                assert int(status) == 0
            else:
                K.attention_mma_ext(q_rows, pool, o, part_acc, part_ml, items, plan.n_small, 16, positions, tables, tpr,
                                    **opts, tok_nsplit=tns, counters=counters)
            assert int(counters.abs().sum()) == 0
        if plan.n_big and kernel == "tc":
            status = torch.zeros(1, dtype=torch.int32, device="cuda")
            tc = {k: v for k, v in opts.items() if k not in ("dv", "kparts")}
            K.attention_tc_ext(q_rows, pool, o, items.view(-1)[plan.n_small * 8:], plan.n_big, positions, tables,
                               status=status, part_acc=part_acc, part_ml=part_ml, tok_part_row=tpr, **tc)
            assert int(status) == 0
            if plan.big_split:
                K.attention_combine(part_acc, part_ml, tpr, tns, o, nq=nq, d=dv, **gate)
        elif plan.n_big:
            K.attention_mma_ext(q_rows, pool, o, part_acc, part_ml, items.view(-1)[plan.n_small * 8:], plan.n_big, 64,
                                positions, tables, tpr, **opts)
    else:
        K.attention_simt(q_rows, pool, o, part_acc, part_ml, items, n, n, positions, tables, tpr, **opts)
        if plan.part_rows:
            K.attention_combine(part_acc, part_ml, tpr, tns, o, nq=nq, d=dv, **gate)
    return o.float().cpu().double(), plan


@pytest.mark.parametrize("dtype,kernel", [(torch.float32, "simt"), (torch.bfloat16, "simt"), (torch.bfloat16, "mma"),
                                          (torch.bfloat16, "tc")])
@pytest.mark.parametrize("page_size,H,G,d,dv,rdim,cap,L", [(16, 4, 2, 32, 48, 8, 30.0, 200), (8, 3, 3, 16, 16, 16, 5.0, 150),
                                                           (16, 2, 1, 64, 128, 32, 0.0, 1300), (32, 8, 1, 24, 40, 0, 50.0, 333),
                                                           (16, 4, 2, 32, 64, 16, 6.0, 200), (32, 6, 3, 64, 128, 64, 30.0, 400)])
def test_score_maps_far_keys_and_the_cap(dtype, kernel, page_size, H, G, d, dv, rdim, cap, L):
    """q, k and v go through the rotate-and-append kernel into shuffled pages in two steps; then a prompt
    portion, a short portion and single decoded tokens attend.  For the probing query one key far back (position
    3, in the first page) is made to stand out in map 1 and another (at a page border) in map 2, each with values
    of its own: a map that reads the other map's keys, a lost far key or a missing cap changes the output by far
    more than the tolerance.  Then the maps are combined (difference, unit norm, gate) and compared again."""
    from mini_hisparse_b200.kernels import api as K
    from mini_hisparse_b200.parts.attention import AttentionShape
    from mini_hisparse_b200.parts.base import Segment

    if kernel == "mma" and not K.attention_mma_ext_supports(d, dv):
        pytest.skip("widths the tensor-core attention does not take")
    M = 2
    # "tc": every q map padded with zeros to the width of a KV head's key row, then plain grouped-query attention
    padded = kernel == "tc"
    if padded and not (M * d == dv and dv in (64, 128) and K.attention_tma_supports(dv, page_size)):
        pytest.skip("the tcgen05 kernel takes key rows as wide as the values, 64 or 128, over pages that divide 64")
    g = torch.Generator().manual_seed(4)
    scale = 2.2 / math.sqrt(d)
    portion = 30
    pages = -(-L // page_size)
    table = torch.randperm(pages + 3, generator=g)[:pages].to(torch.int32)
    pool = torch.full((pages + 3, G * page_size * (M * d + dv)), 1e30).to(dtype).cuda()
    qw, kw, vw = H * M * d, G * M * d, G * dv
    proj = torch.randn(2, L, qw + kw + vw + H + 3, generator=g) * 0.5 ** 0.5   # two split-K parts (unit sum); the gates follow v
    pos = torch.arange(L, dtype=torch.int32)
    inv = torch.tensor([100.0 ** (-2.0 * i / rdim) for i in range(rdim // 2)]) if rdim else None
    q_all = torch.full((L, qw * (M if padded else 1)), 7.0, dtype=dtype, device="cuda")
    for lo, hi in ((0, L - portion), (L - portion, L)):
        pp = proj[:, lo:hi].contiguous().cuda()
        K.rope_append_maps(pp, dev_i(pos[lo:hi]), torch.zeros(hi - lo, dtype=torch.int32, device="cuda"),
                           dev_i(table[None, :]), None if inv is None else inv.cuda(), rdim, True, q_all[lo:hi], pool,
                           nq=H * M, nkv=G, kparts=M, d=d, dv=dv, page_size=page_size, nsplit=2,
                           split_stride=pp.stride(0), q_pad=padded)
    q_rows_all = q_all
    if padded:          # map m of a head sits at the columns of map m, the rest of its row is zero
        wide = q_all.float().cpu().view(L, H, M, M, d)
        assert float(wide[:, :, 0, 1].abs().max()) == 0.0 and float(wide[:, :, 1, 0].abs().max()) == 0.0
        q_all = torch.stack((wide[:, :, 0, 0], wide[:, :, 1, 1]), 2).reshape(L, qw).to(dtype).cuda()
    ps = proj.double().sum(0)
    rot = (lambda t: P.rotate_interleaved(t, pos, rdim, 100.0)) if rdim else (lambda t: t)
    qf = rot(ps[:, :qw].reshape(L, H * M, d)).view(L, H, M, d)
    kf = rot(ps[:, qw:qw + kw].reshape(L, G * M, d)).view(L, G, M, d)
    vf = ps[:, qw + kw:qw + kw + vw].view(L, G, dv)
    pk = pool.float().cpu().view(pages + 3, -1)[table.long()]
    got_k = pk[:, :G * page_size * M * d].reshape(pages, G, page_size, M, d).permute(0, 2, 1, 3, 4).reshape(-1, G, M, d)[:L]
    got_v = pk[:, G * page_size * M * d:].reshape(pages, G, page_size, dv).permute(0, 2, 1, 3).reshape(-1, G, dv)[:L]
    # float32 angles: position times frequency is rounded to 24 bits, so far positions turn by up to 1e-4 radians less or more
    tol = max(5e-6, 3e-7 * L) if dtype == torch.float32 else 0.02
    assert float((got_k.double() - kf).abs().max()) < tol * float(kf.abs().max())
    assert float((got_v.double() - vf).abs().max()) < tol * float(vf.abs().max())
    assert float((q_all.float().cpu().double().view(L, H, M, d) - qf).abs().max()) < tol * float(qf.abs().max())
    # make two far keys stand out in the CACHE (and in the plain copy), one per map
    kc, vc = got_k.double().clone(), got_v.double().clone()
    qc = q_all.float().cpu().double().view(L, H, M, d)
    probe = L - 5
    lift = math.log(L / 50)
    far = {0: 3, 1: page_size * (1 + (L // 3) // page_size)}        # map -> position of its key (the second: first of a page)
    for m, p_ in far.items():
        page, within = int(table[p_ // page_size]), p_ % page_size
        flat = pool[page].float()
        for gk in range(G):
            qd = qc[probe, gk * (H // G), m]
            key = (qd * ((9.0 + lift) / (scale * float(qd @ qd)))).to(dtype).double()
            kc[p_, gk, m] = key
            a = (gk * page_size + within) * M * d + m * d
            flat[a:a + d] = key.float().cuda()
            vc[p_, gk] = 3.0 if m == 0 else -2.0
            b = G * page_size * M * d + (gk * page_size + within) * dv
            flat[b:b + dv] = 3.0 if m == 0 else -2.0
        pool[page] = flat.to(dtype)
    right = plain_maps_attention(qc, kc, vc, torch.arange(L), scale, cap)
    # sharp: the maps swapped, the far keys hidden, or the cap left out are far from right at the probe
    swapped = plain_maps_attention(qc, kc.flip(2), vc, torch.arange(L), scale, cap)
    hidden = plain_maps_attention(qc[probe:probe + 1], kc[4:], vc[4:], torch.tensor([probe - 4]), scale, cap)
    assert float((swapped[probe] - right[probe]).abs().max()) > 0.2
    assert float((hidden[0] - right[probe]).abs().max()) > 0.2
    if cap and cap < 9.0:
        assert float((plain_maps_attention(qc, kc, vc, torch.arange(L), scale, 0.0)[probe] - right[probe]).abs().max()) > 0.2
    shape = AttentionShape(H, G, None, {"mma": 64, "simt": 16}.get(kernel, 0))
    opts = dict(nq=H * M, nkv=G, d=d, dv=dv, page_size=page_size, window=0, scale=scale, kparts=M, softcap=cap)
    if padded:
        shape = AttentionShape(H * M, G, None, 128)
        opts.update(d=M * d, kparts=1)
    bound = 3e-6 if dtype == torch.float32 else 0.02
    whole = None
    for seg, rows in ((Segment("a", 0, L - portion, portion, 0), torch.arange(L - portion, L)),     # a portion of a prompt
                      (Segment("a", 0, L - 9, 9, 0), torch.arange(L - 9, L)),                        # a short portion
                      (Segment("a", 0, probe, 1, 0), torch.tensor([probe])),                         # decoded alone
                      (Segment("a", 0, 0, 20, 0), torch.arange(0, 20))):                             # the first tokens
        got, plan = attend(K, kernel, dtype, shape, [seg], q_rows_all[rows].contiguous(), pool, table, (H * M, dv),
                           torch.float32, **opts)
        assert float((got.view(-1, H, M, dv) - right[rows]).abs().max()) < bound * float(right.abs().max())
        if seg.count == portion:
            whole = got
    # the maps into one output: a1 - lambda a2, over its root mean square, times (1 - init), times the head's gate
    lam, init, eps = 0.37, 0.6, 1e-5
    rows = torch.arange(L - portion, L)
    gates = proj[:, rows][:, :, qw + kw + vw:qw + kw + vw + H].contiguous().cuda()
    out = torch.empty(portion, H * dv, dtype=dtype, device="cuda")
    K.maps_combine(whole.float().cuda().view(portion, H, M, dv), lam, eps, 1 - init, out, gate=gates[0], gate_nsplit=2,
                   gate_split_stride=gates.stride(0))
    o = whole.view(portion, H, M, dv)[:, :, 0] - lam * whole.view(portion, H, M, dv)[:, :, 1]
    ref = P.unit_rms(o, eps) * (1 - init) * torch.sigmoid(gates.double().sum(0).cpu())[:, :, None]
    assert float((out.float().cpu().double().view(portion, H, dv) - ref).abs().max()) < \
        (3e-6 if dtype == torch.float32 else 0.01) * float(ref.abs().max())


@pytest.mark.parametrize("dtype,kernel", [(torch.float32, "simt"), (torch.bfloat16, "simt"), (torch.bfloat16, "mma"),
                                          (torch.bfloat16, "tc")])
@pytest.mark.parametrize("page_size,window,H,d,dr,rank", [(16, 48, 4, 24, 8, 40), (8, 33, 20, 16, 16, 32), (16, 300, 3, 12, 4, 12),
                                                          (32, 150, 8, 64, 32, 96), (16, 1150, 2, 32, 16, 64), (16, 1, 2, 8, 2, 24),
                                                          (16, 90, 40, 16, 16, 48), (16, 1150, 4, 64, 32, 96)])
def test_latent_rows_at_the_windows_edges(dtype, kernel, page_size, window, H, d, dr, rank):
    """The latent rows go through their kernel (unit norm with weight, the shared key part rotated) into shuffled
    pages in two steps, q's unrotated parts are carried into the latent space by one small matrix per head; then a
    prompt portion, a short portion and single decoded tokens attend with the row as key and value.  The row just
    inside the window and the row just outside it are made to stand out for the probing query: a window that is
    one off changes the output by far more than the tolerance."""
    from mini_hisparse_b200.kernels import api as K
    from mini_hisparse_b200.parts.attention import AttentionShape
    from mini_hisparse_b200.parts.base import Segment

    width = rank + dr
    if kernel == "mma" and not K.attention_mma_ext_supports(width, rank):
        pytest.skip("widths the tensor-core attention does not take")
    if kernel == "tc" and not (width in (64, 128) and K.attention_tma_supports(width, page_size)):
        pytest.skip("the tcgen05 kernel takes rows 64 or 128 wide over pages that divide 64")
    vw = width if kernel == "tc" else rank          # the tcgen05 tiles take the whole row as the value
    g = torch.Generator().manual_seed(5)
    L = 200 if window < 1000 else 1300
    scale = 2.2 / math.sqrt(width)
    eps = 1e-5
    portion = 30
    pages = -(-L // page_size)
    table = torch.randperm(pages + 3, generator=g)[:pages].to(torch.int32)
    pool = torch.full((pages + 3, page_size, width), 1e30).to(dtype).cuda()
    qw = H * (d + dr)
    proj = torch.randn(2, L, qw + width + H + 5, generator=g) * 0.5 ** 0.5     # two split-K parts whose sum has unit variance
    cw = 1 + 0.1 * torch.randn(rank, generator=g)
    uk = torch.randn(H, d, rank, generator=g) / math.sqrt(d)          # k_h = uk[h] @ c ... stored [H * d, rank]
    pos = torch.arange(L, dtype=torch.int32)
    inv = torch.tensor([100.0 ** (-2.0 * i / dr) for i in range(dr // 2)])
    q_plain = torch.empty(L, H, d, dtype=dtype, device="cuda")
    q_full = torch.zeros(L, H, width, dtype=dtype, device="cuda")
    for lo, hi in ((0, L - portion), (L - portion, L)):
        pp = proj[:, lo:hi].contiguous().cuda()
        K.latent_prep(pp, cw.cuda(), eps, dev_i(pos[lo:hi]), torch.zeros(hi - lo, dtype=torch.int32, device="cuda"),
                      dev_i(table[None, :]), inv.cuda(), False, q_plain[lo:hi], q_full[lo:hi], pool, heads=H, d=d, dr=dr,
                      rank=rank, page_size=page_size, nsplit=2, split_stride=pp.stride(0))
    K.head_linear(q_plain, uk.transpose(1, 2).contiguous().to(dtype).cuda(), q_full[:, :, :rank])
    ps = proj.double().sum(0)
    qh = ps[:, :qw].view(L, H, d + dr)
    c = P.unit_rms(ps[:, qw:qw + rank], eps) * cw.double()
    kr = P.rotate_half_split(ps[:, None, qw + rank:qw + width], pos, dr, 100.0)[:, 0]
    rows_ref = torch.cat((c, kr), 1)
    got_rows = pool.float().cpu()[table.long()].reshape(-1, width)[:L].double()
    # float32 angles: position times frequency is rounded to 24 bits, so far positions turn by up to 1e-4 radians less or more
    tol = max(5e-6, 3e-7 * L) if dtype == torch.float32 else 0.02
    assert float((got_rows - rows_ref).abs().max()) < tol * float(rows_ref.abs().max())
    q_ref = torch.cat((torch.einsum("thd,hdr->thr", qh[..., :d], uk.to(dtype).double()),
                       P.rotate_half_split(qh[..., d:], pos, dr, 100.0)), -1)
    got_q = q_full.float().cpu().double()
    assert float((got_q - q_ref).abs().max()) < (max(tol, 1e-5) if dtype == torch.float32 else 0.03) * float(q_ref.abs().max())
    # the window's edges at the probe stand out in the cache
    rc = got_rows.clone()
    probe = L - 5
    lift = max(0.0, math.log(window / 50))
    inside, outside = probe - window + 1, probe - window
    for p_, val, score in ((inside, 3.0, 8.0 + lift), (outside, -3.0, 10.0 + lift)):
        if p_ >= 0 and p_ != probe:
            qd = got_q[probe, 0]
            row = (qd * (score / (scale * float(qd @ qd)))).to(dtype).double()
            ones = torch.ones(rank, dtype=torch.float64)       # the row is its own value: mark it, across the query
            row[:rank] += val * (ones - qd[:rank] * (float(ones @ qd[:rank]) / float(qd[:rank] @ qd[:rank])))
            row = row.to(dtype).double()
            rc[p_] = row
            pool[int(table[p_ // page_size]), p_ % page_size] = row.to(dtype).cuda()

    def plain(win):
        diff = torch.arange(L)[:, None] - torch.arange(L)[None, :]
        seen = (diff >= 0) & (diff < win)
        s = torch.einsum("thw,lw->thl", got_q, rc) * scale
        return torch.softmax(s.masked_fill(~seen[:, None, :], -math.inf), -1) @ rc[:, :rank]

    right = plain(window)
    if inside >= 0 and window > 1:
        for wrong in (plain(window + 1), plain(window - 1)):
            assert float((wrong[probe] - right[probe]).abs().max()) > 0.2
    g0 = qw + width
    shape = AttentionShape(H, 1, window, {"tc": 128, "mma": 64, "simt": 16}[kernel])
    bound = 3e-6 if dtype == torch.float32 else 0.02
    for seg, rows in ((Segment("a", 0, L - portion, portion, 0), torch.arange(L - portion, L)),
                      (Segment("a", 0, L - 9, 9, 0), torch.arange(L - 9, L)),
                      (Segment("a", 0, probe, 1, 0), torch.tensor([probe])),
                      (Segment("a", 0, L - 1, 1, 0), torch.tensor([L - 1])),
                      (Segment("a", 0, 0, 20, 0), torch.arange(0, 20))):
        gates = proj[:, rows][:, :, g0:g0 + H].contiguous().cuda()
        opts = dict(nq=H, nkv=1, d=width, dv=vw, page_size=page_size, window=window, scale=scale, shared_kv=True,
                    gate=gates[0], gate_nsplit=2, gate_split_stride=gates.stride(0), gate_per_head=True)
        got, plan = attend(K, kernel, dtype, shape, [seg], q_full[rows].contiguous(), pool, table, (H, vw), dtype, **opts)
        if kernel == "tc" and window > 1000 and seg.count > 16 and seg.start > 1000:
            assert plan.big_split                     # few tiles far into a long window: their keys are split
        ref = right[rows] * torch.sigmoid(gates.double().sum(0).cpu())[:, :, None]
        assert float((got[..., :rank] - ref).abs().max()) < bound * float(right.abs().max())


# ---- the model through the step function -----------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(CONFIGS))
def test_every_schedule_agrees_with_the_plain_model(models, name, dtype):
    """Whole prompts; most of a prompt and then its tail token by token, three requests side by side
    (captured graphs, the window passes over decoded tokens); portions of changing size down to two
    tokens; mixed batches with up to four live requests over a pool that holds no more than they need,
    so that pages and slots are used again (freed pages are poisoned).  Every position is compared."""
    folder, cfg, w = models[name]
    reqs = requests_for(cfg, [150, 1, 23, 97, 64, 2, 131])
    refs = {rid: P.forward(cfg, w, toks).float() for rid, toks in reqs.items()}
    page = {"A": 16, "B": 8, "C": 32, "D": 16}[name]
    whole = None
    for steps in (S.whole(reqs), S.tail_one_by_one(reqs, tail=45), S.changing_portions(reqs), S.mixed(reqs, seed=3)):
        got, runner, cache = run_steps(folder, dtype, steps, page_size=page)
        check_against_plain(got, refs, dtype)
        whole = whole or got
        worst = max(row_rms_error(got[rid], whole[rid]) for rid in reqs)
        print(f"{name} {dtype}: worst row against the whole prompt {worst:.3g}")
        assert worst < (F32_ROW if dtype == "float32" else BF16_CUT)
    assert all(g["pages_reused"] > 0 for g in cache["page_groups"])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_far_keys_and_key_splits(tmp_path, dtype):
    """A request of 700 tokens under causal maps and a latent window of 2,000: decoded tokens and short portions
    far into it have their keys split over several CTAs, whose parts are merged (the gate comes after the merge);
    every key back to the first stays visible."""
    from mini_hisparse_b200 import write_random_model

    cfg = model(120, 128, [layer("attention", maps(4, 2, 32, 64, 16, scale=0.25), ff=192),
                           layer("latent_attention", latent(4, 32, 16, 32, 48, 2000, scale=0.2))], loop=(0, 2, 2))
    write_random_model(cfg, 31, tmp_path, dtype=torch.bfloat16, matrix_std=0.15)
    cfg, w = P.load_folder(tmp_path)
    reqs = requests_for(cfg, [700], seed=70)
    refs = {rid: P.forward(cfg, w, toks).float() for rid, toks in reqs.items()}
    whole = None
    for steps in (S.whole(reqs), S.tail_one_by_one(reqs, tail=40), S.changing_portions(reqs, sizes=(530, 2, 7, 64, 3, 2))):
        got, stats, pages = run_steps(tmp_path, dtype, steps)
        check_against_plain(got, refs, dtype)
        whole = whole or got
        assert row_rms_error(got["r0"], whole["r0"]) < (F32_ROW if dtype == "float32" else BF16_CUT)


def test_the_plain_model_is_sensitive_to_what_the_tests_are_for(models):
    """A window one key off, maps that are not subtracted as they should be, a cap left out, a pass that does not
    see the embedding output again, one pass fewer: each moves the plain model's logits by far more than the
    float32 tolerance, so the comparison above would show them."""
    folder, cfg, w = models["A"]
    toks = random_tokens(cfg["vocab"], 90, 5)
    right = P.forward(cfg, w, toks)
    rms = float(right.pow(2).mean().sqrt())

    def moved(cfg2=None, w2=None):
        return float((P.forward(cfg2 or cfg, w2 or w, toks) - right).pow(2).mean().sqrt()) / rms

    for li, delta in ((0, 1), (0, -1), (2, 1), (2, -1)):
        c = copy.deepcopy(cfg)
        c["layers"][li]["mixer"]["mask"]["size"] += delta
        assert moved(c) > 25 * F32_ROW
    for change in (lambda c: c["layers"][1]["mixer"].update(diff=0.45), lambda c: c["layers"][3]["mixer"].update(softcap=6.0),
                   lambda c: c["loop"].update(times=2), lambda c: c["layers"][1]["mixer"]["rot"].update(dims=6)):
        c = copy.deepcopy(cfg)
        change(c)
        assert moved(c) > 25 * F32_ROW
    w2 = dict(w)
    w2["loop.in"] = w["loop.in"].clone()
    w2["loop.in"][:, cfg["width"]:] = 0            # the embedding output drops out of the passes' inputs
    assert moved(w2=w2) > 25 * F32_ROW
    w2 = dict(w)
    w2["l1.mix.lq2"] = w["l1.mix.lq2"] + 0.5
    assert moved(w2=w2) > 25 * F32_ROW


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_and_a_slot_used_again(models, dtype):
    """A short prompt, then 260 tokens one by one (several windows and many pages long), two requests side by
    side; then their slots and pages serve new requests."""
    folder, cfg, w = models["A"]
    reqs = requests_for(cfg, [270, 265], seed=40)
    refs = {rid: P.forward(cfg, w, toks).float() for rid, toks in reqs.items()}
    steps = S.tail_one_by_one(reqs, tail=260, together=2)
    again = requests_for(cfg, [50, 31], seed=60)
    again = {f"again_{k}": v for k, v in again.items()}
    refs.update({rid: P.forward(cfg, w, toks).float() for rid, toks in again.items()})
    steps += S.changing_portions(again, sizes=(2, 29, 1, 7))
    got, runner, cache = run_steps(folder, dtype, steps, max_requests=2)
    check_against_plain(got, refs, dtype)
    assert runner["graph_steps"] > 200


def test_batches_of_unequal_requests_equal_each_alone(models):
    """float32: a request's logits in a mixed batch equal those it gets alone, to rounding."""
    folder, cfg, w = models["C"]
    reqs = requests_for(cfg, [140, 3, 77, 30], seed=9)
    alone, _, _ = run_steps(folder, "float32", S.whole(reqs), page_size=16)
    mixed, _, _ = run_steps(folder, "float32", S.mixed(reqs, seed=11, tail=20), page_size=16)
    for rid in reqs:
        assert row_rms_error(mixed[rid], alone[rid]) < F32_ROW


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_engine(models, dtype):
    """Engine.add_request / run: admission, portions under a token budget, decoding, finishing.  float32 tokens
    equal the plain model's; in bfloat16 every token is the plain model's choice for the engine's own history,
    or loses to it by less than rounding."""
    from mini_hisparse_b200 import Engine, load_model

    folder, cfg, w = models["A"]
    model_ = load_model(folder, dtype=dtype)
    engine = Engine(model_, num_pages=40, page_size=16, max_requests=3, max_tokens_per_step=48, graph_after=2)
    prompts = requests_for(cfg, [70, 9, 33], seed=80)
    for rid, p in prompts.items():
        engine.add_request(rid, p, max_new_tokens=12)
    out = engine.run()
    engine.cache.assert_invariants()
    for rid, p in prompts.items():
        assert len(out[rid]) == 12
        if dtype == "float32":
            assert out[rid] == P.generate(cfg, w, p, 12)
        else:
            seq = list(p)
            for tok in out[rid]:
                logits = P.forward(cfg, w, seq)[-1]
                assert float(logits.max() - logits[tok]) < 0.05 * float(logits.abs().max())
                seq.append(tok)


def test_command_line_demo_with_a_dotivik_config(capsys):
    """`demo --config configs/dotivik-demo.json`: random weights, three requests through Engine and scheduler."""
    from pathlib import Path

    import mini_hisparse_b200
    from mini_hisparse_b200 import cli

    config = Path(mini_hisparse_b200.__file__).parent / "configs" / "dotivik-demo.json"
    assert cli.main(["demo", "--config", str(config), "--dtype", "bfloat16", "--requests", "3", "--prompt-tokens", "70",
                     "--max-new-tokens", "6"]) == 0
    report = json.loads(capsys.readouterr().out)
    assert [r["generated_tokens"] for r in report["requests"].values()] == [6, 6, 6]
    assert {g["window"] for g in report["cache"]["page_groups"]} == {None, 48}


def test_trace_run_picks_the_model_by_its_config(models, tmp_path):
    """bin/trace_run on a Dotivik folder: the same program, cache and step function as for every model."""
    folder, cfg, w = models["B"]
    reqs = requests_for(cfg, [60, 21], seed=90)
    refs = {rid: P.forward(cfg, w, toks).float() for rid, toks in reqs.items()}
    steps = S.mixed(reqs, seed=1, tail=10)
    run = TraceRun(folder, "float32", tmp_path / "out", S.peak_tokens(steps), page_size=16, extra=("--poison",))
    got = {}
    for entries, end in steps:
        logits = run.step(entries, end)
        row = 0
        for e in entries:
            got.setdefault(e["id"], []).append(logits[row: row + len(e["want"])])
            row += len(e["want"])
    assert run.close() == 0
    check_against_plain({k: torch.cat(v) for k, v in got.items()}, refs, "float32")
