"""Zadunex without a GPU: its configuration, its plan, the cache's storage for it, and the engine's step
logic over it with the kernels replaced by their plain torch restatement (tests/torch_ops.py), against
the plain implementation (tests/plain_zadunex.py)."""

import copy

import pytest
import torch

from torch_ops import TorchOps
from zadunex_helpers import CONFIGS, assert_logits, config, plain_logits, prompts, write_folder


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = tmp_path_factory.mktemp("zadunex")
    return {name: write_folder(root / name, name) for name in CONFIGS}


def cpu_engine(folder, **kw):
    from kernel_rush_kawk_b200 import Engine

    args = dict(dtype="float32", device="cpu", ops=TorchOps(torch.float32), max_tokens=1024, max_slots=5,
                max_context=512, use_cuda_graphs=False)
    args.update(kw)
    return Engine(folder, **args)


def test_config_reads_back_and_is_found_by_its_name(folders):
    from kernel_rush_kawk_b200 import ZadunexConfig, read_config

    for name in CONFIGS:
        arch, cfg = read_config(folders[name])
        assert arch.name == "Zadunex" and isinstance(cfg, ZadunexConfig)
        assert ZadunexConfig.from_dict(cfg.to_dict()) == cfg
        assert cfg.streams == CONFIGS[name]["streams"] and cfg.logit_scale == CONFIGS[name].get("logit_scale", 1.0)
    assert config("za").layer_runs() == [0, 1, 2, 1, 2, 1, 2, 3]
    assert config("zb").layer_runs() == [0, 1, 2] and config("zc").layer_runs() == [0, 1, 0, 1]
    assert config("ze").layer_runs() == [0, 0]


def test_one_stream_with_or_without_hyper_connection_weights_is_read_off_the_checkpoint(folders):
    from kernel_rush_kawk_b200 import ZadunexConfig
    from kernel_rush_kawk_b200.weights.loader import checkpoint_shapes

    raw = copy.deepcopy(CONFIGS["zd"])
    raw.pop("hyper")
    cfg = ZadunexConfig.from_dict(raw)
    assert cfg.hyper and not cfg.with_tensor_shapes(checkpoint_shapes(folders["zd"])).hyper
    assert config("zc").with_tensor_shapes(checkpoint_shapes(folders["zc"])).hyper


@pytest.mark.parametrize("damage, word", [
    (lambda c: c["layers"][1].__setitem__("type", "conv"), "type"),
    (lambda c: c["layers"][1]["mixer"].__setitem__("kv_heads", 3), "multiple"),
    (lambda c: c["layers"][1]["mixer"]["rot"].__setitem__("dims", 7), "even"),
    (lambda c: c["layers"][0]["mixer"].pop("state"), "state"),
    (lambda c: c["layers"][0]["mixer"].__setitem__("groups", 3), "multiple"),
    (lambda c: c["layers"][0]["mixer"].__setitem__("norm_groups", 5), "norm_groups"),
    (lambda c: c["layers"][1]["mlp"]["router"].__setitem__("top", 9), "top"),
    (lambda c: c["layers"][0]["mlp"].pop("limit"), "limit"),
    (lambda c: c["layers"][0].__setitem__("mlp", {"kind": "sparse"}), "kind"),
    (lambda c: c["loop"].__setitem__("stop", 9), "loop"),
    (lambda c: c.__setitem__("streams", 0), "streams"),
    (lambda c: c.pop("norm"), "norm"),
    (lambda c: c.__setitem__("layers", []), "layers"),
])
def test_config_faults_are_named(damage, word):
    from kernel_rush_kawk_b200 import ConfigError, ZadunexConfig

    raw = copy.deepcopy(CONFIGS["za"])
    damage(raw)
    with pytest.raises(ConfigError, match=word):
        ZadunexConfig.from_dict(raw)


def test_plan_names_every_tensor_and_every_run_of_a_layer_keeps_storage_of_its_own():
    from kernel_rush_kawk_b200.cache import SequenceCache
    from kernel_rush_kawk_b200.config.registry import get_architecture
    from kernel_rush_kawk_b200.engine.model import PartTree
    from kernel_rush_kawk_b200.parts import KVNeed, StateNeed

    cfg = config("za")
    plan = get_architecture("Zadunex").plan(cfg)
    tree = PartTree(plan)
    names = tree.expected_tensors()
    assert tuple(names["l0.mix.in"].shape) == (2 * 64 + 2 * 2 * 24 + 4, 64)
    assert tuple(names["l0.mix.conv"].shape) == (64 + 2 * 2 * 24, 4) and tuple(names["l2.mix.conv"].shape) == (64 + 2 * 16, 3)
    assert tuple(names["l1.mix.q.norm"].shape) == (4 * 16,) and tuple(names["l1.mix.k.norm"].shape) == (2 * 16,)
    assert tuple(names["l1.mix.v.b"].shape) == (2 * 24,) and "l1.mix.sink" not in names
    assert tuple(names["l0.hc2.mix"].shape) == (2, 2) and tuple(names["l3.hc1.out"].shape) == (2,)
    assert "l3.norm2" not in names and "l3.hc2.in" not in names and "l3.norm2" in plan.ignored
    assert "l1.mlp.router.b" not in names and "l1.mlp.e4.down" in names and "l0.mlp.gate" in names
    assert [e.layer for e in plan.schedule] == [0, 1, 2, 1, 2, 1, 2, 3]
    needs = tree.cache_needs()
    assert needs[0] == (StateNeed((4, 24, 16), "float32"), StateNeed((3, 64 + 96), "compute"))
    assert needs[1] == needs[3] == needs[5] == KVNeed(2, 16, None, 24)
    assert needs[2] == needs[4] == (StateNeed((2, 16, 32), "float32"), StateNeed((2, 64 + 32), "compute"))
    cache = SequenceCache(needs, 256, 2, 256, "cpu", torch.float32)
    views = [cache.view(r) for r in range(len(needs))]
    assert len({v.k.data_ptr() for v in (views[1], views[3], views[5])}) == 3  # one layer, three runs, three caches
    assert len({v[0].state.data_ptr() for v in (views[2], views[4], views[6])}) == 3
    assert views[2][1].state.shape[1:] == (2, 96)


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

    eng = cpu_engine(folders["za"], max_slots=4)
    for round_ in range(2):  # the second round's sequences get slots whose states and pages the first left behind
        seqs = prompts("za", [40, 1, 75, 13], seed=3 + round_)
        slots = [eng.cache.alloc() for _ in seqs]
        heads = [len(ids) - 2 if len(ids) > 2 else len(ids) for ids in seqs]
        first = eng.step([StepEntry(s, ids[:n], [n - 1]) for s, ids, n in zip(slots, seqs, heads)])
        for i, (ids, n) in enumerate(zip(seqs, heads)):
            assert_logits(first[i:i + 1], plain_logits(folders["za"], ids)[n - 1:n], "float32", f"batched prompt {i}")
        live = [(s, ids) for s, ids in zip(slots, seqs) if len(ids) > 2]
        for back in (2, 1):
            got = eng.step([StepEntry(s, [ids[-back]], [0]) for s, ids in live])
            for i, (s, ids) in enumerate(live):
                ref = plain_logits(folders["za"], ids)
                assert_logits(got[i:i + 1], ref[len(ids) - back:len(ids) - back + 1], "float32", f"batched token of sequence {i}")
        for s in slots:
            eng.cache.free(s)
        eng.cache.check()
