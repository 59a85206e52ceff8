"""The Gamilorn design without a GPU: configuration and registry, weights, the cache manager's
share (values of another size than keys, pages of kept first keys, composite caches), and the
engine's host logic with the kernel wrappers replaced by plain PyTorch restatements (fixture
``torch_ops``), against the plain implementation of ``tests/plain_gamilorn.py``."""

import copy
import json

import pytest
import torch

from deterministic_inference_b200.cache.manager import CacheManager
from deterministic_inference_b200.config import EngineConfig, SamplingParams
from deterministic_inference_b200.config.gamilorn_config import GamilornConfig
from deterministic_inference_b200.config.model_config import ConfigError
from deterministic_inference_b200.engine import Engine, ModelRunner, SequenceInput
from deterministic_inference_b200.models.registry import build_model, config_from_dir
from deterministic_inference_b200.parts.spec import CompositeSpec, PagedKVSpec, StateSpec
from deterministic_inference_b200.weights.loader import WeightsError, load_weights
from tests import gamilorn_util as gu
from tests import plain_gamilorn as pg


@pytest.fixture(scope="module")
def model_dirs(tmp_path_factory):
    return {name: gu.write_tiny(name, tmp_path_factory.mktemp(f"gamilorn_{name}")) for name in gu.CONFIGS}


# ---- configuration, registry, weights ---------------------------------------------------------

def test_the_registry_picks_the_design_by_its_name_and_reads_every_size(model_dirs):
    cfg = config_from_dir(model_dirs["g1"])
    assert isinstance(cfg, GamilornConfig)
    raw = gu.CONFIGS["g1"]["config"]
    assert (cfg.vocab, cfg.width, cfg.max_positions) == (raw["vocab"], raw["width"], raw["max_positions"])
    assert cfg.norm_eps == raw["norm"]["eps"] and cfg.logit_softcap == raw["logit_softcap"]
    plan = cfg.plan()
    assert [l.feed_forward.kind for l in plan.layers] == ["dense_mlp", "none", "dense_mlp"]
    left = plan.layers[2].mixer.params["branches"][0].params
    assert (left["num_heads"], left["num_kv_heads"], left["head_dim"], left["v_head_dim"]) == (3, 1, 8, 40)
    assert (left["window"], left["keep_first"], left["scale"]) == (5, 9, 0.4)
    assert plan.layers[0].mixer.params["scales"] == [0.9, 1.3]
    assert GamilornConfig.from_dict(cfg.to_dict()).to_dict() == cfg.to_dict()


def test_the_decay_rank_comes_from_the_checkpoint(model_dirs, tmp_path):
    raw = json.loads((model_dirs["g1"] / "config.json").read_text())
    for layer in raw["layers"]:
        del layer["mixer"]["right"]["decay_rank"]       # a published config.json does not carry it
    d = tmp_path / "m"
    d.mkdir()
    (d / "config.json").write_text(json.dumps(raw))
    (d / "model.safetensors").write_bytes((model_dirs["g1"] / "model.safetensors").read_bytes())
    cfg = config_from_dir(d)
    assert [l["mixer"]["right"]["decay_rank"] for l in cfg.layers] == [4, 8, 3]


def test_a_preset_and_the_command_line_write_a_model_folder_the_registry_reads_back(tmp_path):
    from deterministic_inference_b200.__main__ import main
    from deterministic_inference_b200.config import preset

    cfg = preset("gamilorn_tiny")
    assert isinstance(cfg, GamilornConfig) and len(cfg.layers) == 3
    assert main(["random", "--preset", "gamilorn_tiny", "--seed", "4", "--out", str(tmp_path / "m")]) == 0
    back = config_from_dir(tmp_path / "m")
    assert back.to_dict() == cfg.to_dict()
    model = build_model(back, torch.bfloat16, "cpu")
    tensors = load_weights(tmp_path / "m", model.tensor_specs(), model.plan, torch.bfloat16, "cpu")
    assert tensors["l1.mix.right.w1"].shape == (8, 128) and "l1.norm2" not in tensors
    assert tensors["l0.norm1"].dtype == torch.float32 and tensors["l0.mix.left.q"].dtype == torch.bfloat16


@pytest.mark.parametrize("edit, text", [
    (lambda c: c.pop("width"), "width"),
    (lambda c: c["layers"][0].__setitem__("type", "serial"), "type"),
    (lambda c: c["layers"][0]["mixer"]["left"].__setitem__("kv_heads", 3), "multiple"),
    (lambda c: c["layers"][0]["mixer"]["left"]["mask"].__setitem__("size", 0), "mask.size"),
    (lambda c: c["layers"][0]["mlp"].__setitem__("kind", "experts"), "mlp.kind"),
    (lambda c: c.__setitem__("layers", []), "no layers"),
    (lambda c: c["layers"][1]["mixer"]["right"].pop("decay_rank"), "rank of the decay map"),
])
def test_a_configuration_that_cannot_run_is_refused_with_the_reason(edit, text):
    cfg = copy.deepcopy(gu.CONFIGS["g1"]["config"])
    edit(cfg)
    with pytest.raises(ConfigError, match=text):
        GamilornConfig.from_dict(cfg)


def test_the_loader_names_what_a_checkpoint_lacks(model_dirs, tmp_path):
    from safetensors.torch import load_file, save_file
    tensors = load_file(str(model_dirs["g3"] / "model.safetensors"))
    del tensors["l0.mix.left.pb"]
    tensors["l1.mix.right.w0"] = tensors["l1.mix.right.w0"][:-1].contiguous()
    d = tmp_path / "m"
    d.mkdir()
    (d / "config.json").write_text((model_dirs["g3"] / "config.json").read_text())
    save_file(tensors, str(d / "model.safetensors"))
    cfg = config_from_dir(d)
    model = build_model(cfg, torch.float32, "cpu")
    with pytest.raises(WeightsError) as e:
        load_weights(d, model.tensor_specs(), model.plan, torch.float32, "cpu")
    assert "l0.mix.left.pb" in str(e.value) and "l1.mix.right.w0" in str(e.value)


# ---- cache manager ----------------------------------------------------------------------------------

def test_pages_of_kept_first_keys_stay_when_the_window_passes():
    spec = PagedKVSpec(2, 8, window=20, v_head_dim=12, keep_first=18)
    cm = CacheManager({0: spec}, num_pages=12, page_size=8, max_reqs=3, max_seq_len=88, allocate_device=False)
    (g,) = cm.page_groups.values()
    s = cm.allocate_slot()
    cm.allocate(s, 80)
    assert cm.release_passed(s, 80) == 4
    # positions 0..17 are kept: pages 0, 1, 2 stay; a query at 80 reads keys from 61 on: page 7 on
    assert [p != 0 for p in g.pages[s]] == [True, True, True, False, False, False, False, True, True, True]
    cm.check_invariants()
    t = cm.allocate_slot()
    cm.allocate(t, 32)              # the freed pages are handed out again
    assert set(g.pages[t]) <= set(range(1, 12)) and not set(g.pages[t]) & set(p for p in g.pages[s] if p)
    cm.release_slot(s)
    cm.release_slot(t)
    cm.check_invariants()
    assert g.num_free == 11


def test_a_composite_cache_lives_in_its_members_groups():
    kv = PagedKVSpec(2, 8, window=None, v_head_dim=4)
    st = StateSpec((3, 5, 5), "float32")
    cm = CacheManager({0: CompositeSpec((kv, st)), 1: CompositeSpec((kv, st)), 2: st}, num_pages=6,
                      page_size=4, max_reqs=3, max_seq_len=20, dtype=torch.float32, device="cpu")
    assert len(cm.page_groups) == 1 and len(cm.state_groups) == 1
    (g,) = cm.page_groups.values()
    assert tuple(g.pool.shape) == (2, 6, 2 * 4 * (8 + 4))         # a page: keys, then values
    (sg,) = cm.state_groups.values()
    assert tuple(sg.array.shape) == (3, 3, 3, 5, 5)

    from types import SimpleNamespace
    meta = SimpleNamespace(slot_mapping=None)
    Step = SimpleNamespace(groups={g.key: meta})
    v = cm.view(1, Step)
    assert v.members[0].kv.data_ptr() == g.pool[1].data_ptr() and v.members[0].attention_meta is meta
    assert v.members[1].state.data_ptr() == sg.array[1].data_ptr()
    assert cm.view(2, Step).state.data_ptr() == sg.array[2].data_ptr()


# ---- the engine's host logic on the CPU -------------------------------------------------------------

def runner_for(model_dir, page, pool, **kw):
    return ModelRunner(EngineConfig(model_path=str(model_dir), dtype="float32", device="cpu",
                                    kv_pool_tokens=pool, page_size=page, max_reqs=3, max_seq_len=pool,
                                    debug_checks=True, **kw))


@pytest.mark.parametrize("name", ["g1", "g3"])
def test_cuttings_batches_and_reused_slots_on_cpu(name, model_dirs, torch_ops):
    d = model_dirs[name]
    cfg, w = pg.read_model_dir(d, torch.float32)
    toks, other, third = gu.requests(cfg["vocab"], [70, 41, 26], 3)
    ref, ref_other, ref_third = (pg.forward(cfg, w, t) for t in (toks, other, third))
    r = runner_for(d, gu.CONFIGS[name]["page_size"], pool=208)
    tol = dict(atol=3e-4, rtol=1e-4)

    s = r.cache.allocate_slot()
    logits, _ = r.step([SequenceInput(s, toks, 0, [0, 5, 69])])
    torch.testing.assert_close(logits, ref[[0, 5, 69]], **tol)
    r.cache.release_slot(s)

    # portions down to two tokens beside a request that decodes token by token; the first
    # request's slot is the one just freed: its state must start from zero again
    s, o = r.cache.allocate_slot(), r.cache.allocate_slot()
    r.step([SequenceInput(o, other[:20], 0, [])])
    c, oc = 0, 20
    for n in (13, 2, 7, 2, 25, 5, 16):
        entries = [SequenceInput(s, toks[c:c + n], c, list(range(n)))]
        if oc < len(other):
            entries.insert(0, SequenceInput(o, other[oc:oc + 1], oc, [0]))
        logits, batch = r.step(entries)
        torch.testing.assert_close(logits[batch.logit_rows[-1]], ref[c:c + n], **tol)
        if len(entries) == 2:
            torch.testing.assert_close(logits[batch.logit_rows[0]], ref_other[oc:oc + 1], **tol)
            oc += 1
        c += n
    assert c == 70
    r.cache.release_slot(s)
    # a third request takes over slot and pages while the other one goes on
    s = r.cache.allocate_slot()
    logits, batch = r.step([SequenceInput(s, third, 0, list(range(26))), SequenceInput(o, other[oc:oc + 1], oc, [0])])
    torch.testing.assert_close(logits[batch.logit_rows[0]], ref_third, **tol)
    torch.testing.assert_close(logits[batch.logit_rows[1]], ref_other[oc:oc + 1], **tol)
    r.cache.release_slot(s)
    r.cache.release_slot(o)
    r.cache.check_invariants()


def test_greedy_generation_through_the_entry_point_on_cpu(model_dirs, torch_ops):
    d = model_dirs["g1"]
    cfg, w = pg.read_model_dir(d, torch.float32)
    prompts = gu.requests(cfg["vocab"], [3, 20, 9], 7)
    want = [pg.generate(cfg, w, p, 8) for p in prompts]
    eng = Engine(EngineConfig(model_path=str(d), dtype="float32", device="cpu", kv_pool_tokens=96, page_size=16,
                              max_reqs=2, max_seq_len=64, max_prefill_tokens=12, cuda_graphs=False,
                              async_scheduling=False))
    outs = eng.generate(prompts, SamplingParams(max_new_tokens=8, ignore_eos=True))
    assert [o.token_ids for o in outs] == want
    eng.cache.check_invariants()
