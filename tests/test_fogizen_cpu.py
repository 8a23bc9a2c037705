"""Fogizen without a GPU: its configuration, its plan, the cache's storage for it, and the engine's step
logic over it with the kernels replaced by their plain torch restatement (tests/torch_ops.py), against
the plain implementation (tests/plain_fogizen.py)."""

import copy

import pytest
import torch

from fogizen_helpers import CONFIGS, assert_logits, config, plain_logits, prompts, write_folder
from torch_ops import TorchOps


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = tmp_path_factory.mktemp("fogizen")
    return {name: write_folder(root / name, name) for name in CONFIGS}


def cpu_engine(folder, **kw):
    from kernel_rush_kawk_b200 import Engine

    args = dict(dtype="float32", device="cpu", ops=TorchOps(torch.float32), max_tokens=1024, max_slots=5,
                max_context=512, use_cuda_graphs=False)
    args.update(kw)
    return Engine(folder, **args)


def test_config_reads_back_and_is_found_by_its_name(folders):
    from kernel_rush_kawk_b200 import FogizenConfig, read_config

    for name in CONFIGS:
        arch, cfg = read_config(folders[name])
        assert arch.name == "Fogizen" and isinstance(cfg, FogizenConfig)
        assert FogizenConfig.from_dict(cfg.to_dict()) == cfg
        assert cfg.buckets == CONFIGS[name]["embedding"]["bigram"]["buckets"]
    assert config("fa").layers[2]["mixer"]["left"]["rot"] is None and config("fb").layers[2]["mixer"]["left"]["mask"] is None
    assert config("fa").layers[0]["mixer"]["left"]["rot"]["scaling"]["factor"] == 2.0


def test_the_decays_rank_is_read_off_the_checkpoint(folders):
    from kernel_rush_kawk_b200.weights.loader import checkpoint_shapes

    raw = copy.deepcopy(CONFIGS["fa"])
    for layer in raw["layers"]:
        layer["mixer"]["right"].pop("rank")
    from kernel_rush_kawk_b200 import FogizenConfig
    cfg = FogizenConfig.from_dict(raw).with_tensor_shapes(checkpoint_shapes(folders["fa"]))
    assert [layer["mixer"]["right"]["rank"] for layer in cfg.layers] == [8, 12, 4]


@pytest.mark.parametrize("damage, word", [
    (lambda c: c["layers"][1].__setitem__("type", "conv"), "type"),
    (lambda c: c["layers"][0]["mixer"]["left"].__setitem__("kv_heads", 3), "multiple"),
    (lambda c: c["layers"][0]["mixer"]["left"]["rot"].__setitem__("dims", 7), "even"),
    (lambda c: c["layers"][0]["mixer"]["left"]["rot"]["scaling"].__setitem__("factor", 0), "positive"),
    (lambda c: c["layers"][0]["mixer"]["left"]["mask"].__setitem__("size", 0), "size"),
    (lambda c: c["layers"][0]["mixer"].pop("right"), "right"),
    (lambda c: c["layers"][0]["mlp"]["router"].__setitem__("top", 5), "top"),
    (lambda c: c["layers"][0]["mlp"]["router"]["groups"].__setitem__("count", 4), "groups"),
    (lambda c: c["layers"][0]["mlp"]["router"]["groups"].__setitem__("keep", 4), "groups"),
    (lambda c: c["layers"][1]["mlp"].pop("ff"), "ff"),
    (lambda c: c["layers"][1].__setitem__("mlp", {"kind": "sparse"}), "kind"),
    (lambda c: c["embedding"]["bigram"].pop("buckets"), "buckets"),
    (lambda c: c["embedding"]["bigram"].__setitem__("mul_prev", -1), "mul_prev"),
    (lambda c: c.pop("norm"), "norm"),
    (lambda c: c.__setitem__("layers", []), "layers"),
])
def test_config_faults_are_named(damage, word):
    from kernel_rush_kawk_b200 import ConfigError, FogizenConfig

    raw = copy.deepcopy(CONFIGS["fa"])
    damage(raw)
    with pytest.raises(ConfigError, match=word):
        FogizenConfig.from_dict(raw)


def test_plan_names_every_tensor_and_every_layer_keeps_five_kinds_of_storage(folders):
    from safetensors import safe_open
    from kernel_rush_kawk_b200.cache import SequenceCache
    from kernel_rush_kawk_b200.config.registry import get_architecture
    from kernel_rush_kawk_b200.engine.model import PartTree
    from kernel_rush_kawk_b200.parts import KVNeed, StateNeed

    cfg = config("fa")
    plan = get_architecture("Fogizen").plan(cfg)
    tree = PartTree(plan)
    names = tree.expected_tensors()
    with safe_open(str(folders["fa"] / "model.safetensors"), framework="pt") as f:
        stored = {k: tuple(f.get_slice(k).get_shape()) for k in f.keys()}
    assert {k: tuple(v.shape) for k, v in names.items()} == stored
    assert tuple(names["bigram"].shape) == (54, 64) and tuple(names["l0.shift"].shape) == (64,)
    assert tuple(names["l0.mix.left.q.norm"].shape) == (16,) and tuple(names["l0.mix.left.talk"].shape) == (4, 4)
    assert tuple(names["l0.mix.left.g"].shape) == (4, 64) and tuple(names["l0.mix.left.out"].shape) == (64,)
    assert tuple(names["l1.mix.right.w1"].shape) == (12, 64) and tuple(names["l1.mlp.act"].shape) == (2,)
    assert tuple(names["l0.mlp.correction"].shape) == (6,) and "l0.mlp.router.b" not in names and "l0.norm2" not in names
    assert not any(k.startswith("l2.mlp") for k in names) and plan.layers[2].feed_forward is None
    assert all(layer.feed_forward_norm is None for layer in plan.layers)
    needs = tree.cache_needs()
    assert len(needs) == 4 and needs[3] == StateNeed((1,), "int32")  # the embedding's last token
    assert needs[0] == (StateNeed((64,), "float32"), KVNeed(2, 16, None, 32), StateNeed((3, 16, 16), "float32"),
                        StateNeed((64,), "float32"))
    cache = SequenceCache(needs, 256, 2, 256, "cpu", torch.float32)
    shift, kv, state, last = cache.view(1)
    assert shift.state.data_ptr() != last.state.data_ptr() and shift.state.shape == last.state.shape == (2, 64)
    assert kv.k.shape[1:] == (2, 64, 24) and kv.v.shape[1:] == (2, 64, 8) and state.state.shape == (2, 1, 48, 48)
    assert cache.view(3).state.dtype == torch.int32


@pytest.mark.parametrize("name", list(CONFIGS))
def test_whole_prompts_portions_and_single_tokens_agree_with_the_plain_implementation(folders, name):
    from kernel_rush_kawk_b200 import StepEntry

    eng = cpu_engine(folders[name])
    ids = prompts(name, [90])[0]
    ref = plain_logits(folders[name], ids)
    for pieces in ([90], [40, 2, 3, 45], [70] + [1] * 20):
        slot = eng.cache.alloc()
        got, start = [], 0
        for n in pieces:
            got.append(eng.step([StepEntry(slot, ids[start:start + n], list(range(n)))]))
            start += n
        eng.cache.free(slot)
        assert_logits(torch.cat(got), ref, "float32", f"{name}, pieces {pieces[:4]}")
    eng.cache.check()


def test_unequal_batch_against_each_alone_and_a_slot_used_again(folders):
    from kernel_rush_kawk_b200 import StepEntry

    eng = cpu_engine(folders["fa"], max_slots=4)
    for round_ in range(2):  # the second round's sequences get slots whose states and pages the first left behind
        seqs = prompts("fa", [40, 1, 75, 13], seed=3 + round_)
        slots = [eng.cache.alloc() for _ in seqs]
        heads = [len(ids) - 2 if len(ids) > 2 else len(ids) for ids in seqs]
        first = eng.step([StepEntry(s, ids[:n], [n - 1]) for s, ids, n in zip(slots, seqs, heads)])
        for i, (ids, n) in enumerate(zip(seqs, heads)):
            assert_logits(first[i:i + 1], plain_logits(folders["fa"], ids)[n - 1:n], "float32", f"batched prompt {i}")
        live = [(s, ids) for s, ids in zip(slots, seqs) if len(ids) > 2]
        for back in (2, 1):
            got = eng.step([StepEntry(s, [ids[-back]], [0]) for s, ids in live])
            for i, (s, ids) in enumerate(live):
                ref = plain_logits(folders["fa"], ids)
                assert_logits(got[i:i + 1], ref[len(ids) - back:len(ids) - back + 1], "float32", f"batched token of sequence {i}")
        for s in slots:
            eng.cache.free(s)
        eng.cache.check()


def test_random_weights_by_preset_name_build_a_model():
    from kernel_rush_kawk_b200 import FogizenConfig
    from kernel_rush_kawk_b200.config.registry import get_architecture, preset_config
    from kernel_rush_kawk_b200.engine.model import PartTree

    assert "fogizen_tiny" in FogizenConfig.preset_names()
    for name in FogizenConfig.preset_names():
        cfg = preset_config(name)
        tree = PartTree(get_architecture("Fogizen").plan(cfg))
        assert "l0.mix.left.talk" in tree.expected_tensors()


def test_command_line_writes_a_preset_as_a_model_folder(tmp_path, capsys):
    from kernel_rush_kawk_b200 import cli, read_config

    assert cli.main(["write-random", "--preset", "fogizen_tiny", "--seed", "1", "--out", str(tmp_path / "m")]) == 0
    arch, cfg = read_config(tmp_path / "m")
    assert arch.name == "Fogizen" and len(cfg.layers) == 3
    eng = cpu_engine(tmp_path / "m", max_tokens=256, max_context=256)
    steps = list(eng.generate([[5, 6, 7], [9]], 3))
    assert len(steps) == 3 and all(len(s) == 2 for s in steps)


# ----------------------------------------------------------------------------------------------
# the parts alone, with the kernels' plain torch restatement, against the plain functions
# ----------------------------------------------------------------------------------------------

def _rand(shape, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(shape, generator=g) * scale


def _runtime():
    from kernel_rush_kawk_b200.engine.model import Runtime

    return Runtime(torch.device("cpu"), torch.float32, TorchOps(torch.float32))


def _context(rt, slots, starts, token_lists, cache):
    from kernel_rush_kawk_b200.engine.step import BatchMeta, StepContext

    meta = BatchMeta(sum(len(t) for t in token_lists), len(slots), 0, rt.device)
    meta.fill(slots, starts, token_lists, [])
    return StepContext(rt.ops, meta, cache)


def _run_mixer(part, rt, h, pieces):
    from kernel_rush_kawk_b200.cache import SequenceCache

    cache = SequenceCache([part.cache_need()], 512, 1, 512, rt.device, torch.float32)
    slot = cache.alloc()
    got, start = [], 0
    for n in pieces:
        cache.reserve(slot, start + n)
        cache.sync()
        got.append(part.forward(_context(rt, [slot], [start], [[0] * n], cache), h[start:start + n], cache.view(0)))
        cache.advance(slot, n)
        start += n
    return torch.cat(got)


def test_the_whole_mixer_of_a_layer_in_pieces_against_the_plain_functions():
    """The shifted input, the two mixers side by side, their norms and the half sum, as the plan builds them."""
    import plain_fogizen as plain
    from kernel_rush_kawk_b200.config.registry import get_architecture
    from kernel_rush_kawk_b200.parts import mixer_class

    cfg = config("fa")
    spec = get_architecture("Fogizen").plan(cfg).layers[0].mixer
    part = mixer_class(spec.kind)(dict(spec.params))
    w = {key: _rand(tuple(t.shape), 10 + i, 0.3) + (1.0 if t.role == "gain" else 0.0)
         for i, (key, t) in enumerate(part.tensor_specs().items())}
    w["inner.left.talk"] = 0.6 * torch.eye(4) + _rand((4, 4), 3, 0.3)
    rt = _runtime()
    part.bind(w, rt)
    T = 45
    n = _rand((T, 64), 5)
    ref = {spec.tensors[k]: v.double() for k, v in w.items()}
    nd = n.double()
    s = nd + (plain.previous_rows(nd) - nd) * ref["l0.shift"]
    want = plain.mixer(s, ref, "l0.mix.", CONFIGS["fa"]["layers"][0]["mixer"] | {"right": {"heads": 3, "dim": 16}}, cfg.eps,
                       torch.arange(T))
    for pieces in ([T], [9, 1, 2, 33], [20] + [1] * 25):
        got = _run_mixer(part, rt, n, pieces)
        assert (got.double() - want).abs().max() < 2e-4 * want.abs().max(), f"pieces {pieces[:4]}"


@pytest.mark.parametrize("shape", [(64, 6, 2, 3, 2, 24, 1.5), (96, 4, 4, 4, 4, 16, 0.7), (50, 9, 2, 3, 2, 11, 1.0), (64, 8, 3, 2, 1, 40, 2.5)])
def test_routing_within_groups_and_the_dense_activation_against_the_plain_functions(shape):
    import plain_fogizen as plain
    from types import SimpleNamespace
    from kernel_rush_kawk_b200.parts import DenseMLP, RoutedExperts

    C, E, top, count, keep, F, scale = shape
    rt = _runtime()
    part = RoutedExperts({"hidden": C, "experts": E, "top": top, "intermediate": F, "scoring": "sigmoid_groups",
                          "groups": count, "keep_groups": keep, "route_scale": scale})
    w = {"router": _rand((E, C), 1, 0.5), "correction": _rand((E,), 2, 0.6) - 0.5}
    for e in range(E):
        w.update({f"e{e}.gate": _rand((F, C), 10 + 3 * e, 0.3), f"e{e}.up": _rand((F, C), 11 + 3 * e, 0.3),
                  f"e{e}.down": _rand((C, F), 12 + 3 * e, 0.3)})
    part.bind(w, rt)
    h = _rand((30, C), 7, 1.5)
    ref = {k: v.double() for k, v in w.items()}
    router = {"experts": E, "top": top, "scale": scale, "groups": {"count": count, "keep": keep}}
    want = plain.routed_ff(h.double(), ref, "", {"router": router})
    got = part.forward(SimpleNamespace(ops=rt.ops, batch=SimpleNamespace(is_decode=False)), h)
    assert (got.double() - want).abs().max() < 1e-4 * want.abs().max()
    dense = DenseMLP({"hidden": C, "intermediate": F, "activation": "xielu"})
    wd = {"up": _rand((F, C), 3, 0.5), "down": _rand((C, F), 4, 0.3), "act": torch.tensor([0.4, -1.2])}
    dense.bind(wd, rt)
    want = plain.dense_ff(h.double(), {k: v.double() for k, v in wd.items()}, "")
    got = dense.forward(SimpleNamespace(ops=rt.ops), h)
    assert (got.double() - want).abs().max() < 1e-4 * want.abs().max()
