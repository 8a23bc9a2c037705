"""Fogizen on the GPU: every mechanism's kernels alone against the plain functions of
tests/plain_fogizen.py, then the model through the engine: whole prompts, portions, single tokens,
unequal batches, reused slots, long decoding, greedy generation and trace replay."""

import io
import json
from types import SimpleNamespace

import pytest
import torch

import plain_fogizen as plain
from fogizen_helpers import CONFIGS, assert_logits, plain_logits, prompts, write_folder

pytestmark = pytest.mark.gpu

DTYPES = (torch.float32, torch.bfloat16)
PART_TOL = {torch.float32: 3e-5, torch.bfloat16: 5e-2}


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = tmp_path_factory.mktemp("fogizen_gpu")
    return {name: write_folder(root / name, name) for name in CONFIGS}


def runtime(dtype, head_dims=()):
    """``head_dims``: the head sizes whose tensor-core attention libraries the test's steps of many tokens may use."""
    from kernel_rush_kawk_b200.csrc import load_kernels
    from kernel_rush_kawk_b200.engine.model import Runtime

    return Runtime(torch.device("cuda:0"), dtype, load_kernels(tuple(head_dims)))


def rand(shape, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(shape, generator=g) * scale


def context(rt, slots, starts, token_lists, cache):
    from kernel_rush_kawk_b200.engine.step import BatchMeta, StepContext

    meta = BatchMeta(sum(len(t) for t in token_lists), len(slots), 0, rt.device)
    meta.fill(slots, starts, token_lists, [])
    return StepContext(rt.ops, meta, cache)


def close(got, ref, dtype, what):
    got, ref = got.detach().double().cpu(), ref.detach().double().cpu()
    assert got.shape == ref.shape, f"{what}: shape {tuple(got.shape)} vs {tuple(ref.shape)}"
    assert torch.isfinite(got).all(), f"{what}: non-finite values"
    err = (got - ref).abs().max().item()
    tol = PART_TOL[dtype] * ref.abs().max().item()
    assert err <= tol, f"{what}: max |d| = {err:.3e} > {tol:.3e}; first bad row {int(((got - ref).abs() > tol).any(-1).nonzero()[0])}"


def run_part(part, rt, h, pieces, dtype, prior=(), forward=None):
    """One sequence through a part that keeps storage, cut into ``pieces``; ``prior``: sequences that used (and
    gave back) the slot before."""
    from kernel_rush_kawk_b200.cache import SequenceCache

    cache = SequenceCache([part.cache_need()], 2048, 1, 2048, rt.device, dtype)
    for seq, cuts in list(prior) + [(h, pieces)]:
        slot = cache.alloc()
        got, start = [], 0
        for n in cuts:
            cache.reserve(slot, start + n)
            cache.sync()
            ctx = context(rt, [slot], [start], [[0] * n], cache)
            got.append(part.forward(ctx, seq[start:start + n].to(dtype).cuda(), cache.view(0)))
            cache.advance(slot, n)
            start += n
        cache.free(slot)
    rt.ops.check()
    return torch.cat(got)


def as_path(w, dtype):
    """The tensors as the path stores them, and the same values in float64 for the plain functions."""
    stored = {k: v.to(torch.bfloat16) for k, v in w.items()}  # checkpoints hold bfloat16
    return {k: v.to(dtype).cuda() for k, v in stored.items()}, {k: v.double() for k, v in stored.items()}


# ----------------------------------------------------------------------------------------------
# each mechanism alone
# ----------------------------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("vocab, width, buckets, mul_prev, mul_cur", [(211, 64, 53, 7, 3), (301, 50, 1, 5, 9),
                                                                      (50000, 24, 100003, 2000003, 1999993)])
def test_pair_hash_embedding_over_pieces_and_reused_slots(dtype, vocab, width, buckets, mul_prev, mul_cur):
    from kernel_rush_kawk_b200.cache import SequenceCache
    from kernel_rush_kawk_b200.parts import BigramEmbedding

    rt = runtime(dtype)
    part = BigramEmbedding({"vocab": vocab, "hidden": width, "buckets": buckets, "mul_prev": mul_prev, "mul_cur": mul_cur})
    w = {"table": rand((vocab, width), 1), "pairs": rand((buckets + 1, width), 2)}
    assert {k: tuple(s.shape) for k, s in part.tensor_specs().items()} == {k: tuple(v.shape) for k, v in w.items()}
    dev, ref = as_path(w, dtype)
    part.bind(dev, rt)
    cache = SequenceCache([part.cache_need()], 256, 2, 256, rt.device, dtype)
    g = torch.Generator().manual_seed(3)
    e = {"buckets": buckets, "mul_prev": mul_prev, "mul_cur": mul_cur}
    for round_ in range(2):  # the second round's sequences start on slots that still hold the first round's last tokens
        seqs = [torch.randint(vocab - 40, vocab, (n,), generator=g).tolist() for n in (23, 9)]
        slots = [cache.alloc() for _ in seqs]
        got = [[], []]
        for cuts in ([(0, 7), (0, 1)], [(7, 9), (1, 2)], [(9, 10), (2, 9)], [(10, 23), None]):
            live = [i for i, c in enumerate(cuts) if c is not None]
            ctx = context(rt, [slots[i] for i in live], [cuts[i][0] for i in live], [seqs[i][cuts[i][0]:cuts[i][1]] for i in live], cache)
            out = part.forward(ctx, cache.view(0))
            assert out.dtype == torch.float32
            row = 0
            for i in live:
                n = cuts[i][1] - cuts[i][0]
                got[i].append(out[row:row + n])
                row += n
        for i, ids in enumerate(seqs):
            want = plain.embed(ids, ref["table"], ref["pairs"], e)
            assert (torch.cat(got[i]).double().cpu() - want).abs().max() < 1e-6, f"round {round_}, sequence {i}"
        for s in slots:
            cache.free(s)
    rt.ops.check()


@pytest.mark.parametrize("dtype", DTYPES)
def test_token_shift_keeps_the_last_row_of_every_sequence(dtype):
    rt = runtime(dtype)
    C = 50
    h = [rand((n, C), 10 + i).to(dtype) for i, n in enumerate((17, 5))]
    mu = rand((1, C), 3).cuda()
    state = torch.zeros((3, C), device="cuda")
    state[2] = 7.0  # a slot that nobody uses keeps what it holds
    got = [[], []]
    for cuts in ([(0, 6), (0, 1)], [(6, 7), (1, 2)], [(7, 17), (2, 5)]):
        rows = torch.cat([h[i][a:b] for i, (a, b) in enumerate(cuts)]).cuda()
        ctx = context(rt, [1, 0], [c[0] for c in cuts], [[0] * (b - a) for a, b in cuts], None)
        out = rt.ops.token_shift(rows, state, mu, ctx.batch, store=True)[0]
        got[0].append(out[:cuts[0][1] - cuts[0][0]])
        got[1].append(out[cuts[0][1] - cuts[0][0]:])
    for i in range(2):
        x = h[i].double()
        want = x + (plain.previous_rows(x) - x) * mu.double().cpu()
        close(torch.cat(got[i]), want, dtype, f"sequence {i}")
    assert torch.equal(state[1].cpu(), h[0][-1].float()) and torch.equal(state[0].cpu(), h[1][-1].float())
    assert (state[2] == 7.0).all()


LEFT_SHAPES = [  # hidden, heads, kv heads, dim, vdim, block, rotated, base, factor
    (64, 4, 2, 16, 32, 10, 8, 100.0, 2.0),
    (48, 2, 2, 24, 8, 37, 24, 5000.0, 1.0),
    (50, 3, 3, 6, 5, 3, 4, 7.0, 1.25),
    (96, 6, 1, 32, 32, 100, 16, 15000.0, 4.0),
    (64, 8, 2, 64, 64, 64, 64, 500.0, 8.0),
    (32, 1, 1, 16, 24, None, 0, 1.0, 1.0),
    (40, 5, 1, 10, 6, 128, 10, 50.0, 2.0),
    (64, 13, 13, 16, 16, 70, 16, 100.0, 1.0),    # a prime number of heads: one block of thirteen warps
    (64, 32, 8, 32, 32, 64, 16, 100.0, 2.0),     # bfloat16 prompts: two blocks of sixteen heads share a tile
    (48, 20, 4, 48, 48, 90, 24, 1000.0, 1.0),    # two blocks of ten heads, five heads a kv head
]


def left_part(shape, dtype, rt, seed=70):
    from kernel_rush_kawk_b200.parts import SinkWindowAttention

    C, H, G, D, Dv, block, rot, base, factor = shape
    part = SinkWindowAttention({"hidden": C, "heads": H, "kv_heads": G, "dim": D, "vdim": Dv, "scale": 0.3, "window": None,
                                "rot_dims": rot, "rot_base": base, "rot_factor": factor, "rot_pairs": True, "chunk": block,
                                "talk": True, "sink": True, "gate": "head", "bias": True, "qk_norm": "head", "eps": 1e-5})
    w = {"q": rand((H * D, C), seed, 0.5), "k": rand((G * D, C), seed + 1, 0.5), "v": rand((G * Dv, C), seed + 2, 0.3),
         "o": rand((C, H * Dv), seed + 3, 0.3), "q.b": rand((H * D,), seed + 4, 0.5), "k.b": rand((G * D,), seed + 5, 0.5),
         "v.b": rand((G * Dv,), seed + 6, 0.5), "q.norm": 1 + rand((D,), seed + 7, 0.3), "k.norm": 2 + rand((D,), seed + 8, 0.3),
         "talk": 0.6 * torch.eye(H) + rand((H, H), seed + 9, 0.4), "sink": rand((H,), seed + 10, 2.0),
         "g": rand((H, C), seed + 11, 0.5)}
    assert {k: tuple(s.shape) for k, s in part.tensor_specs().items()} == {k: tuple(v.shape) for k, v in w.items()}
    dev, ref = as_path(w, dtype)
    part.bind(dev, rt)
    m = {"heads": H, "kv_heads": G, "dim": D, "vdim": Dv, "scale": 0.3, "mask": {"size": block} if block else None,
         "rot": {"dims": rot, "base": base, "scaling": {"factor": factor}} if rot else None}
    return part, ref, m


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", LEFT_SHAPES)
def test_attention_with_mixed_scores_whole_in_pieces_and_token_by_token(dtype, shape):
    rt = runtime(dtype, (shape[3],) if shape[3] == shape[4] and shape[3] % 16 == 0 else ())
    part, ref, m = left_part(shape, dtype, rt)
    assert part.attention_head_dims() == ((shape[3],) if shape[3] == shape[4] and shape[3] % 16 == 0 else ())
    T = 150
    h = rand((T, shape[0]), 5, 1.0).to(dtype)
    want = plain.left_branch(h.double(), ref, "", m, 1e-5, torch.arange(T))
    other = rand((70, shape[0]), 6, 1.0).to(dtype)
    for pieces, prior in (([T], ()), ([63, 2, 1, 64, 20], [(other, [70])]), ([T - 40] + [1] * 40, ())):
        close(run_part(part, rt, h, pieces, dtype, prior), want, dtype, f"attention {shape}, pieces {pieces[:5]}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads, kv, dim, vdim, block", [(4, 2, 16, 8, 50), (3, 1, 8, 40, 64), (6, 6, 32, 32, 200), (2, 1, 32, 32, None),
                                                          (12, 4, 64, 64, 100), (24, 6, 32, 32, 80)])
def test_a_planted_key_shows_just_inside_a_block_and_not_just_outside(dtype, heads, kv, dim, vdim, block):
    """One key is made to stand out for a query: as the block's first key it takes the whole softmax, as the last key
    of the block before it must not be seen at all. Prompts and single tokens, page borders, a far key without blocks.
    (Twenty-four heads: in bfloat16 two thread blocks share a tile's heads and read one another's scores.)"""
    from kernel_rush_kawk_b200.cache import SequenceCache
    from kernel_rush_kawk_b200.parts import KVNeed

    rt = runtime(dtype, (dim,) if dim == vdim and dim % 16 == 0 else ())  # bfloat16 prompts then take the tensor cores
    T = 330
    q = rand((T, heads, dim), 1)
    k = rand((T, kv, dim), 2)
    v = rand((T, kv, vdim), 3)
    talk = 0.8 * torch.eye(heads) + rand((heads, heads), 4, 0.2)
    sink = rand((heads,), 5)
    edges = [block, 2 * block, 3 * block] if block else [64, 128]
    for e in edges:
        if e + 9 >= T:
            continue
        for p, j in ((e + 9, e), (e + 5, e - 1), (e - 1, e - (block or 60))):
            k[j, 0] = 40.0 * q[p, 0] / q[p, 0].norm()  # a score of about 20 |q| against scores of a few
    q, k, v = (t.to(dtype) for t in (q, k, v))
    want = plain.mixed_chunk_attention(q.double(), k.double(), v.double(), 0.5, talk.double(), sink.double(), block)
    cache = SequenceCache([KVNeed(kv, dim, None, None if vdim == dim else vdim)], 1024, 1, 1024, rt.device, dtype)
    inv_freq = torch.zeros(0, device="cuda")
    for pieces in ([T], [block or 64, 1, 1, 61, 2] + [1] * 30 + [T - 95 - (block or 64)], [T - 100] + [1] * 100):
        assert sum(pieces) == T
        slot = cache.alloc()
        got, start = [], 0
        for n in pieces:
            cache.reserve(slot, start + n)
            cache.sync()
            ctx = context(rt, [slot], [start], [[0] * n], cache)
            proj = torch.cat([q[start:start + n].reshape(n, -1), k[start:start + n].reshape(n, -1), v[start:start + n].reshape(n, -1)],
                             dim=1).contiguous().cuda()
            out = torch.empty((n, heads * vdim), dtype=dtype, device="cuda")
            rt.ops.bias_norm_rotate_write(proj, 0, heads * dim, (heads + kv) * dim, heads, kv, dim, vdim, None, None, 0.0,
                                          inv_freq, 0, True, ctx.batch, cache.view(0))
            rt.ops.mixed_attention(proj, 0, heads, dim, vdim, sink.cuda(), talk.cuda().contiguous(), 0.5, block, ctx.batch,
                                   cache.view(0), out, 0, 1.0)
            got.append(out)
            cache.advance(slot, n)
            start += n
        cache.free(slot)
        close(torch.cat(got).view(T, heads, vdim), want, dtype, f"planted keys, block {block}, pieces {pieces[:5]}")
    rt.ops.check()


@pytest.mark.parametrize("dtype", DTYPES)
def test_without_a_mixing_matrix_and_without_a_sink_it_is_plain_attention(dtype):
    from kernel_rush_kawk_b200.cache import SequenceCache
    from kernel_rush_kawk_b200.parts import KVNeed

    rt = runtime(dtype)
    T, H, G, D = 90, 4, 2, 16
    q, k, v = (rand((T, n, D), s).to(dtype) for n, s in ((H, 1), (G, 2), (G, 3)))
    want = plain.mixed_chunk_attention(q.double(), k.double(), v.double(), 0.25, torch.eye(H, dtype=torch.float64),
                                       torch.full((H,), -1e30, dtype=torch.float64), 32)
    cache = SequenceCache([KVNeed(G, D)], 256, 1, 256, rt.device, dtype)
    slot = cache.alloc()
    cache.reserve(slot, T)
    cache.sync()
    ctx = context(rt, [slot], [0], [[0] * T], cache)
    proj = torch.cat([q.reshape(T, -1), k.reshape(T, -1), v.reshape(T, -1)], dim=1).contiguous().cuda()
    out = torch.empty((T, H * D), dtype=dtype, device="cuda")
    rt.ops.bias_norm_rotate_write(proj, 0, H * D, (H + G) * D, H, G, D, D, None, None, 0.0, torch.zeros(0, device="cuda"), 0,
                                  False, ctx.batch, cache.view(0))
    rt.ops.mixed_attention(proj, 0, H, D, D, None, None, 0.25, 32, ctx.batch, cache.view(0), out, 0, 1.0)
    close(out.view(T, H, D), want, dtype, "no mixing, no sink")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hidden, heads, dim, rank", [(64, 3, 16, 8), (50, 1, 7, 3), (96, 5, 8, 6), (64, 2, 48, 12)])
def test_time_mixing_whole_in_pieces_and_token_by_token(dtype, hidden, heads, dim, rank):
    from kernel_rush_kawk_b200.parts import TimeMixWKV

    rt = runtime(dtype)
    part = TimeMixWKV({"hidden": hidden, "heads": heads, "dim": dim, "rank": rank, "eps": 1e-5})
    HN = heads * dim
    w = {"mu." + c: 0.4 + rand((hidden,), 20 + i, 0.3) for i, c in enumerate("rkvgw")}
    w.update({c: rand((HN, hidden), 30 + i, 0.3) for i, c in enumerate("rkvg")})
    w.update({"w1": rand((rank, hidden), 40, 0.3), "w2": rand((HN, rank), 41, 0.5), "w0": rand((HN,), 42, 1.5) - 1.0,
              "u": rand((heads, dim), 43, 0.5), "norm": 1 + rand((HN,), 44, 0.2), "o": rand((hidden, HN), 45, 0.3)})
    assert {k: tuple(s.shape) for k, s in part.tensor_specs().items()} == {k: tuple(v.shape) for k, v in w.items()}
    dev, ref = as_path(w, dtype)
    part.bind(dev, rt)
    T = 140
    h = rand((T, hidden), 7).to(dtype)
    want = plain.right_branch(h.double(), ref, "", {"heads": heads, "dim": dim}, 1e-5)
    other = rand((40, hidden), 8).to(dtype)
    for pieces, prior in (([T], ()), ([33, 2, 1, 64, 40], [(other, [40])]), ([T - 30] + [1] * 30, ())):
        close(run_part(part, rt, h, pieces, dtype, prior), want, dtype, f"time mixing, pieces {pieces[:5]}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width, n", [(64, 2), (50, 2), (33, 3), (2048, 2), (96, 1)])
def test_norms_of_several_outputs_summed(dtype, width, n):
    rt = runtime(dtype)
    ys = [rand((9, width), 10 + b, 1.0 + b).to(dtype) for b in range(n)]
    gains = torch.stack([1 + rand((width,), 20 + b, 0.3) for b in range(n)])
    got = rt.ops.norm_sum([y.cuda() for y in ys], gains.cuda(), 1e-4, 0.5)
    want = 0.5 * sum(plain.rms_norm(y.double(), g.double(), 1e-4) for y, g in zip(ys, gains))
    close(got, want, dtype, f"{n} norms of width {width}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width, inter, rows", [(64, 72, 1), (50, 33, 5), (96, 136, 200)])
@pytest.mark.parametrize("p, q", [(0.3, -0.8), (-2.0, 1.5)])
def test_dense_feed_forward_with_both_sides_of_the_activation(dtype, width, inter, rows, p, q):
    from kernel_rush_kawk_b200.parts import DenseMLP

    rt = runtime(dtype)
    part = DenseMLP({"hidden": width, "intermediate": inter, "activation": "xielu"})
    w = {"up": rand((inter, width), 1, 0.4), "down": rand((width, inter), 2, 0.3), "act": torch.tensor([p, q])}
    assert {k: tuple(s.shape) for k, s in part.tensor_specs().items()} == {k: tuple(v.shape) for k, v in w.items()}
    dev, ref = as_path(w, dtype)
    part.bind(dev, rt)
    h = rand((rows, width), 4, 1.5).to(dtype)
    z = h.double() @ ref["up"].T
    assert (z > 1).any() and (z < -1).any()
    close(part.forward(SimpleNamespace(ops=rt.ops), h.cuda()), plain.dense_ff(h.double(), ref, ""), dtype, "dense feed-forward")


ROUTERS = [  # hidden, experts, top, groups, kept, expert size, scale
    (64, 6, 2, 3, 2, 24, 1.5),
    (96, 4, 4, 4, 4, 16, 0.7),   # groups of one expert, all kept, every expert chosen
    (50, 9, 2, 3, 2, 11, 1.0),
    (64, 8, 3, 2, 1, 40, 2.5),
    (32, 16, 1, 1, 1, 8, 1.0),   # one group
    (64, 40, 6, 8, 3, 16, 2.0),  # more experts than a warp has lanes
]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", ROUTERS)
@pytest.mark.parametrize("rows", [1, 5, 200])
def test_experts_chosen_by_sigmoid_scores_within_the_best_groups(dtype, shape, rows):
    from kernel_rush_kawk_b200.parts import RoutedExperts

    rt = runtime(dtype)
    C, E, top, count, keep, F, scale = shape
    part = RoutedExperts({"hidden": C, "experts": E, "top": top, "intermediate": F, "scoring": "sigmoid_groups",
                          "groups": count, "keep_groups": keep, "route_scale": scale})
    w = {"router": rand((E, C), 1, 0.5), "correction": rand((E,), 2, 0.6) - 0.5}  # choice scores of both signs
    for e in range(E):
        w.update({f"e{e}.gate": rand((F, C), 10 + 3 * e, 0.3), f"e{e}.up": rand((F, C), 11 + 3 * e, 0.3),
                  f"e{e}.down": rand((C, F), 12 + 3 * e, 0.3)})
    assert {k: tuple(s.shape) for k, s in part.tensor_specs().items()} == {k: tuple(v.shape) for k, v in w.items()}
    dev, ref = as_path(w, dtype)
    part.bind(dev, rt)
    h = rand((rows, C), 7, 1.5).to(dtype)
    router = {"experts": E, "top": top, "scale": scale, "groups": {"count": count, "keep": keep}}
    idx, wt = plain.route(h.double(), ref, "", router)
    assert ((torch.sigmoid(h.double() @ ref["router"].T) + ref["correction"]) < 0).any()
    experts, weights, _ = rt.ops.moe_route(h.cuda(), dev["router"], None, top,
                                           sigmoid_groups=(dev["correction"].float(), count, keep, scale))
    if dtype == torch.float32:
        assert torch.equal(experts.cpu().long(), idx), "the chosen experts, in the order of their choice scores"
        assert (weights.double().cpu() - wt).abs().max() < 1e-5
    want = plain.routed_ff(h.double(), ref, "", {"router": router})
    for decode in (False, True):
        ctx = SimpleNamespace(ops=rt.ops, batch=SimpleNamespace(is_decode=decode))
        got = part.forward(ctx, h.cuda())
        if dtype == torch.float32:
            close(got, want, dtype, f"experts {shape}, {rows} rows, single-token step {decode}")
        else:  # a close call may fall the other way in bfloat16: all but a few rows
            bad = ((got.double().cpu() - want).abs() > PART_TOL[dtype] * want.abs().max()).any(-1).sum()
            assert bad <= max(1, rows // 20), f"{int(bad)} of {rows} rows differ"


def test_a_struck_out_group_is_never_chosen_although_its_scores_are_the_largest_left():
    """Four groups of two; the kept groups are the two with the largest sums of their two best choice scores. An expert
    of a lost group has a larger score than the kept groups' second experts, and a kept group's scores are negative."""
    rt = runtime(torch.float32)
    z = torch.tensor([[2.0, 1.9, 3.0, -9.0, 0.5, 0.4, -3.0, -3.5]])
    x = torch.ones((1, 1), device="cuda")
    correction = torch.tensor([0.0, 0.0, 0.0, 0.0, 0.0, 0.0, 0.0, 0.0], device="cuda")
    experts, weights, _ = rt.ops.moe_route(x, z.t().contiguous().cuda(), None, 3, sigmoid_groups=(correction, 4, 2, 2.0))
    s = torch.sigmoid(z[0])
    # group sums: 0: s0 + s1 (largest), 1: s2 + s3, 2: s4 + s5, 3: small -> groups 0 and 2 are kept; expert 2 (the
    # largest single score) is struck out
    assert s[4] + s[5] > s[2] + s[3]
    assert experts[0].tolist() == [0, 1, 4]
    chosen = s[[0, 1, 4]]
    assert torch.allclose(weights[0].cpu(), chosen / chosen.sum() * 2.0, atol=1e-6)
    correction = torch.tensor([-5.0, -5.0, 0.0, 0.0, -5.0, -5.0, -6.0, -6.0], device="cuda")  # negative choice scores win
    experts, weights, _ = rt.ops.moe_route(x, z.t().contiguous().cuda(), None, 3, sigmoid_groups=(correction, 4, 2, 1.0))
    assert experts[0].tolist() == [2, 3, 0]  # groups 1 and 0 are kept (sums near 1 and -8), group 0's scores are negative
    chosen = s[[2, 3, 0]]
    assert torch.allclose(weights[0].cpu(), chosen / chosen.sum(), atol=1e-6)


# ----------------------------------------------------------------------------------------------
# the model through the engine
# ----------------------------------------------------------------------------------------------

def engine(folder, dtype, **kw):
    from kernel_rush_kawk_b200 import Engine

    args = dict(dtype=dtype, max_tokens=4096, max_slots=6, max_context=1024)
    args.update(kw)
    return Engine(folder, **args)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(CONFIGS))
def test_whole_portions_and_single_tokens_through_the_engine(folders, name, dtype):
    from kernel_rush_kawk_b200 import StepEntry

    eng = engine(folders[name], dtype)
    ids = prompts(name, [260])[0]
    ref = plain_logits(folders[name], ids)
    for pieces in ([260], [130, 2, 3, 64, 61], [210] + [1] * 50):
        slot = eng.cache.alloc()
        got, start = [], 0
        for n in pieces:
            got.append(eng.step([StepEntry(slot, ids[start:start + n], list(range(n)))]).clone())
            start += n
        eng.cache.free(slot)
        assert_logits(torch.cat(got), ref, dtype, f"{name} {dtype}, pieces {pieces[:4]}")
    eng.cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_unequal_batches_reused_slots_and_long_decoding(folders, dtype):
    """Five requests of unequal length start together and are decoded together while the shorter ones end; their
    slots, states and pages are then used again by others. Every row against the sequence run alone in the plain
    implementation."""
    from kernel_rush_kawk_b200 import StepEntry

    name = "fa"
    eng = engine(folders[name], dtype, max_slots=5)
    for round_ in range(2):
        lengths = [90, 1, 300, 37, 64] if round_ == 0 else [65, 130, 2]
        tails = [70, 0, 100, 20, 1] if round_ == 0 else [30, 60, 1]
        seqs = prompts(name, lengths, seed=5 + round_)
        slots = [eng.cache.alloc() for _ in seqs]
        heads = [len(ids) - t for ids, t in zip(seqs, tails)]
        first = eng.step([StepEntry(s, ids[:n], [n - 1]) for s, ids, n in zip(slots, seqs, heads)]).clone()
        for i, (ids, n) in enumerate(zip(seqs, heads)):
            assert_logits(first[i:i + 1], plain_logits(folders[name], ids)[n - 1:n], dtype, f"round {round_}, prompt {i}")
        got = {i: [] for i in range(len(seqs))}
        for t in range(max(tails)):
            live = [i for i in range(len(seqs)) if t < tails[i]]
            out = eng.step([StepEntry(slots[i], [seqs[i][heads[i] + t]], [0]) for i in live])
            for row, i in enumerate(live):
                got[i].append(out[row].clone())
            for i in range(len(seqs)):
                if t + 1 == tails[i]:
                    eng.cache.free(slots[i])
        for i, ids in enumerate(seqs):
            if tails[i] == 0:
                eng.cache.free(slots[i])
                continue
            assert_logits(torch.stack(got[i]), plain_logits(folders[name], ids)[heads[i]:], dtype, f"round {round_}, decoded sequence {i}")
        eng.cache.check()
        assert eng.cache.live == 0


def test_greedy_generation_through_the_engines_own_entry(folders):
    """Engine.generate (scheduler, captured single-token steps, selection kernel) against greedy decoding
    with the plain implementation; prompts of unequal length, one of a single token."""
    name = "fb"
    eng = engine(folders[name], "float32", max_tokens=None)
    seqs = prompts(name, [33, 1, 80], seed=9)
    steps = list(eng.generate(seqs, 12))
    assert len(steps) == 12
    cfg, w = plain.read_folder(folders[name], torch.float64)
    for i, ids in enumerate(seqs):
        ids = list(ids)
        for t in range(12):
            logits = plain.forward(cfg, w, ids)[-1]
            best = torch.topk(logits, 2).values
            if best[0] - best[1] < 1e-4:  # too close to call in 32-bit: stop comparing this sequence
                break
            assert steps[t][i] == int(logits.argmax()), f"sequence {i}, new token {t}"
            ids.append(steps[t][i])


def test_trace_replay_serves_the_design(folders, tmp_path):
    """bin/trace_run's program on a small schedule: a batch of prompts, single tokens, a request that ends."""
    from kernel_rush_kawk_b200 import replay

    name = "fc"
    a, b = prompts(name, [70, 9], seed=4)
    lines = [{"step": 0, "entries": [{"id": "a", "tokens": a[:60], "want": [0, 59]}, {"id": "b", "tokens": b[:8], "want": [7]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": [a[60]], "want": [0]}, {"id": "b", "tokens": [b[8]], "want": []}], "end": ["b"]}]
    lines += [{"step": 2 + t, "entries": [{"id": "a", "tokens": [a[61 + t]], "want": [0]}], "end": ["a"] if t == 8 else []} for t in range(9)]
    out = io.StringIO()
    args = replay.build_parser().parse_args(["--model", str(folders[name]), "--dtype", "float32", "--out", str(tmp_path / "o"),
                                             "--max-tokens", "256"])
    assert replay.run(args, stdin=io.StringIO("\n".join(json.dumps(l) for l in lines) + "\n"), stdout=out) == 0
    assert out.getvalue().split() == [w for t in range(11) for w in ("done", str(t))]
    import numpy as np
    ref_a, ref_b = plain_logits(folders[name], a), plain_logits(folders[name], b)
    first = torch.from_numpy(np.fromfile(tmp_path / "o" / "0.f32", dtype="<f4").reshape(3, -1))
    assert_logits(first, torch.stack([ref_a[0], ref_a[59], ref_b[7]]), "float32", "replayed prompts")
    for t in range(10):
        row = torch.from_numpy(np.fromfile(tmp_path / "o" / f"{1 + t}.f32", dtype="<f4").reshape(1, -1))
        assert_logits(row, ref_a[60 + t:61 + t], "float32", f"replayed token {t}")


def test_command_line_writes_a_random_model_and_generates_from_it(tmp_path, capsys):
    """`write-random` (a preset's configuration and seeded weights as a model folder), then `generate` from that folder
    and straight from the preset's name: the same weights, so the same greedy tokens; with a temperature the
    sampler's own seed decides."""
    from kernel_rush_kawk_b200 import cli

    assert cli.main(["write-random", "--preset", "fogizen_tiny", "--seed", "3", "--out", str(tmp_path / "m")]) == 0
    capsys.readouterr()
    common = ["--prompt-ids", "5,6,7,8,9", "--prompt-ids", "11", "--max-new-tokens", "6", "--max-context", "256"]
    assert cli.main(["generate", "--model", str(tmp_path / "m")] + common) == 0
    from_folder = [json.loads(line) for line in capsys.readouterr().out.strip().splitlines()]
    assert cli.main(["generate", "--random", "fogizen_tiny", "--weights-seed", "3"] + common) == 0
    from_preset = [json.loads(line) for line in capsys.readouterr().out.strip().splitlines()]
    assert from_folder == from_preset and [len(r["tokens"]) for r in from_folder] == [6, 6]
    assert cli.main(["generate", "--random", "fogizen_tiny", "--weights-seed", "3", "--temperature", "0.8", "--seed", "4"]
                    + common) == 0
    sampled = [json.loads(line) for line in capsys.readouterr().out.strip().splitlines()]
    assert all(0 <= t < 512 for r in sampled for t in r["tokens"])
