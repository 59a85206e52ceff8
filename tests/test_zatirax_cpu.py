"""The Zatirax design without a GPU: configuration and registry, weights, the cache manager's share
(a chunk mask's pages, a latent cache without values, a cache per pass of a loop), the stretched
rotation frequencies, and the engine's host logic with the kernel wrappers replaced by plain PyTorch
restatements (fixture ``torch_ops``), against the plain implementation of ``tests/plain_zatirax.py``."""

import copy
import json
import math

import pytest
import torch

from deterministic_inference_b200.cache.manager import CacheManager
from deterministic_inference_b200.config import EngineConfig, SamplingParams
from deterministic_inference_b200.config.model_config import ConfigError
from deterministic_inference_b200.config.zatirax_config import ZatiraxConfig
from deterministic_inference_b200.engine import Engine, ModelRunner, SequenceInput
from deterministic_inference_b200.models.registry import build_model, config_from_dir
from deterministic_inference_b200.parts.registry import POSITION_ENCODINGS, BuildContext
from deterministic_inference_b200.parts.spec import PagedKVSpec, PartSpec
from deterministic_inference_b200.weights.loader import WeightsError, load_weights
from tests import plain_zatirax as pz
from tests import zatirax_util as zu


@pytest.fixture(scope="module")
def model_dirs(tmp_path_factory):
    return {name: zu.write_tiny(name, tmp_path_factory.mktemp(f"zatirax_{name}")) for name in zu.CONFIGS}


# ---- configuration, registry, weights ---------------------------------------------------------

def test_the_registry_picks_the_design_by_its_name_and_reads_every_size(model_dirs):
    cfg = config_from_dir(model_dirs["z1"])
    assert isinstance(cfg, ZatiraxConfig)
    raw = zu.CONFIGS["z1"]["config"]
    assert (cfg.vocab, cfg.width, cfg.norm_eps, cfg.embedding_scale) == (150, 64, 2e-5, 3.0)
    assert cfg.loop == (1, 3, 3)
    plan = cfg.plan()
    assert [l.mixer.kind for l in plan.layers] == ["latent_attention", "masked_attention", "masked_attention",
                                                  "latent_attention"]
    assert [l.feed_forward.kind for l in plan.layers] == ["gated_mlp", "none", "gated_mlp", "gated_mlp"]
    a = plan.layers[2].mixer.params
    assert (a["num_heads"], a["num_kv_heads"], a["head_dim"], a["v_head_dim"]) == (3, 1, 32, 16)
    assert (a["mask"], a["mask_size"], a["sink"], a["gate"]) == ("chunk", 13, True, True)
    assert a["position_encoding"].params["rotary_dim"] == 32 and a["position_encoding"].params["scaling"] is None
    b = plan.layers[0].mixer.params
    assert (b["kv_rank"], b["rot_dim"], b["mask"], b["mask_size"]) == (32, 8, "window", 11)
    assert plan.layers[0].feed_forward.params["limit"] == 0.7
    assert ZatiraxConfig.from_dict(cfg.to_dict()).to_dict() == cfg.to_dict()
    assert cfg.to_dict()["layers"] == raw["layers"]


def test_every_run_of_a_layer_has_its_own_cache_and_a_pass_starts_with_its_vector():
    cfg = ZatiraxConfig.from_dict(zu.CONFIGS["z1"]["config"])
    sched = cfg.plan().schedule
    assert [e.layer for e in sched] == [0, 1, 2, 1, 2, 1, 2, 3]
    assert [e.cache for e in sched] == list(range(8))
    assert [e.enter_vector for e in sched] == [None, 0, None, 1, None, 2, None, None]
    # no loop: every layer once, nothing added, no vectors to load
    plan = ZatiraxConfig.from_dict(zu.CONFIGS["z2"]["config"]).plan()
    assert [e.layer for e in plan.schedule] == [0, 1] and plan.stream_addend is None
    # a loop over everything, and one of a single pass
    assert [e.layer for e in ZatiraxConfig.from_dict(zu.CONFIGS["z3"]["config"]).plan().schedule] == [0, 1, 0, 1]
    sched = ZatiraxConfig.from_dict(zu.CONFIGS["z4"]["config"]).plan().schedule
    assert [(e.layer, e.enter_vector) for e in sched] == [(0, None), (1, 0), (2, None)]


@pytest.mark.parametrize("change, text", [
    (lambda c: c["layers"][0].update(type="conv"), "type"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=7), "rot.dims"),
    (lambda c: c["layers"][1]["mixer"].update(kv_heads=3), "multiple"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=6), "rot_dim"),
    (lambda c: c["loop"].update(stop=9), "loop"),
    (lambda c: c["layers"][0]["mlp"].pop("limit"), "limit"),
    (lambda c: c.pop("embedding"), "embedding"),
])
def test_a_configuration_that_cannot_run_is_refused_with_the_reason(change, text):
    raw = copy.deepcopy(zu.CONFIGS["z1"]["config"])
    change(raw)
    with pytest.raises(ConfigError) as e:
        ZatiraxConfig.from_dict(raw)
    assert text in str(e.value)


def test_missing_and_misshapen_tensors_are_listed(model_dirs, tmp_path):
    from safetensors.torch import load_file, save_file
    d = tmp_path / "m"
    d.mkdir()
    (d / "config.json").write_text((model_dirs["z1"] / "config.json").read_text())
    tensors = load_file(str(model_dirs["z1"] / "model.safetensors"))
    del tensors["l1.mix.sink"], tensors["loop.step"]
    tensors["l0.mix.uk"] = tensors["l0.mix.uk"][:, :5].contiguous()
    save_file(tensors, str(d / "model.safetensors"))
    model = build_model(config_from_dir(d), torch.float32, "cpu")
    with pytest.raises(WeightsError) as e:
        load_weights(d, model.tensor_specs(), model.plan, torch.float32, "cpu")
    assert all(n in str(e.value) for n in ("l1.mix.sink", "loop.step", "l0.mix.uk"))


# ---- rotation frequencies ---------------------------------------------------------------------------

@pytest.mark.parametrize("scaling", [None, (8.0, 1.0, 4.0, 512), (2.0, 0.5, 2.0, 32), (4.0, 1.0, 3.0, 64)])
def test_stretched_frequencies(scaling):
    ctx = BuildContext(dtype=torch.float32, device=torch.device("cpu"))
    sc = None if scaling is None else dict(zip(("factor", "low", "high", "original"), scaling))
    rope = POSITION_ENCODINGS.build(PartSpec("rope", dict(head_dim=40, rotary_dim=24, theta=20000.0, scaling=sc)), ctx)
    want = pz.rotary_frequencies(24, 20000.0, sc)
    torch.testing.assert_close(rope.frequencies().double(), want, rtol=1e-7, atol=0)
    if scaling:       # all three branches occur: kept, divided, blended
        plain = pz.rotary_frequencies(24, 20000.0)
        ratio = (want / plain).tolist()
        assert ratio[0] == 1.0 and abs(ratio[-1] - 1 / scaling[0]) < 1e-12
        assert any(1 / scaling[0] + 1e-9 < r < 1 - 1e-9 for r in ratio)


# ---- cache manager ----------------------------------------------------------------------------------

def test_a_chunk_masks_pages_go_back_when_the_chunk_is_left():
    spec = PagedKVSpec(2, 8, window=20, v_head_dim=12, mask="chunk")
    assert spec.group_key() != PagedKVSpec(2, 8, window=20, v_head_dim=12).group_key()
    cm = CacheManager({0: spec}, num_pages=12, page_size=8, max_reqs=3, max_seq_len=88, allocate_device=False)
    (g,) = cm.page_groups.values()
    s = cm.allocate_slot()
    cm.allocate(s, 59)
    # the next query stands at 59, in the chunk 40..59: the pages of positions 0..39 go back
    assert cm.release_passed(s, 59) == 5
    assert [p != 0 for p in g.pages[s]] == [False] * 5 + [True] * 3
    cm.allocate(s, 60)
    # ... at 60 a new chunk begins: only the page that holds 56..63 is still needed
    assert cm.release_passed(s, 60) == 2
    cm.check_invariants()
    # a sliding window of the same size keeps the last 20 keys instead
    cm2 = CacheManager({0: PagedKVSpec(2, 8, window=20)}, num_pages=12, page_size=8, max_reqs=3, max_seq_len=88,
                       allocate_device=False)
    t = cm2.allocate_slot()
    cm2.allocate(t, 60)
    assert cm2.release_passed(t, 60) == 5         # keys from 41 on: pages 0..4 go
    cm.release_slot(s)
    cm.check_invariants()
    assert g.num_free == 11


def test_a_latent_cache_stores_no_values_and_every_pass_has_its_own(model_dirs):
    cfg = config_from_dir(model_dirs["z1"])
    model = build_model(cfg, torch.float32, "cpu")
    specs = model.cache_specs()
    assert len(specs) == 8
    assert specs[0] == PagedKVSpec(1, 32 + 8, window=11, v_head_dim=0)
    assert specs[1] == specs[3] == specs[5] == PagedKVSpec(2, 16, window=16, v_head_dim=24, mask="chunk")
    cm = CacheManager(specs, num_pages=5, page_size=4, max_reqs=3, max_seq_len=16, dtype=torch.float32, device="cpu")
    by_key = {g.key: g for g in cm.page_groups.values()}
    assert tuple(by_key[specs[0].group_key()].pool.shape) == (1, 5, 4 * 40)              # keys only
    assert tuple(by_key[specs[1].group_key()].pool.shape) == (3, 5, 2 * 4 * (16 + 24))   # one pool per pass


# ---- the engine's host logic on the CPU -------------------------------------------------------------

def runner_for(model_dir, page, pool, **kw):
    return ModelRunner(EngineConfig(model_path=str(model_dir), dtype="float32", device="cpu",
                                    kv_pool_tokens=pool, page_size=page, max_reqs=3, max_seq_len=pool,
                                    debug_checks=True, **kw))


@pytest.mark.parametrize("name", list(zu.CONFIGS))
def test_cuttings_batches_and_reused_slots_on_cpu(name, model_dirs, torch_ops):
    d = model_dirs[name]
    cfg, w = pz.read_model_dir(d, torch.float32)
    toks, other, third = zu.requests(cfg["vocab"], [70, 41, 26], 3)
    ref, ref_other, ref_third = (pz.forward(cfg, w, t) for t in (toks, other, third))
    r = runner_for(d, zu.CONFIGS[name]["page_size"], pool=224)
    tol = dict(atol=3e-4, rtol=1e-4)

    s = r.cache.allocate_slot()
    logits, _ = r.step([SequenceInput(s, toks, 0, [0, 5, 69])])
    torch.testing.assert_close(logits, ref[[0, 5, 69]], **tol)
    r.cache.release_slot(s)

    # portions down to two tokens beside a request that decodes token by token, on the slot and
    # pages just freed
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
    s = r.cache.allocate_slot()
    logits, batch = r.step([SequenceInput(s, third, 0, list(range(26))), SequenceInput(o, other[oc:oc + 1], oc, [0])])
    torch.testing.assert_close(logits[batch.logit_rows[0]], ref_third, **tol)
    torch.testing.assert_close(logits[batch.logit_rows[1]], ref_other[oc:oc + 1], **tol)
    r.cache.release_slot(s)
    r.cache.release_slot(o)
    r.cache.check_invariants()


def test_the_stream_after_every_layer_run(model_dirs, torch_ops):
    """The residual stream (pending term added) after each run of a layer, looped ones each time."""
    from deterministic_inference_b200.kernels import ops
    d = model_dirs["z1"]
    cfg, w = pz.read_model_dir(d, torch.float32)
    (toks,) = zu.requests(cfg["vocab"], [19], 5)
    _, want = pz.forward(cfg, w, toks, return_layers=True)
    r = runner_for(d, 16, pool=64)
    seen = []
    r.model.after_layer = lambda e, hidden, residual: seen.append(residual + torch_kernel_plain(hidden))
    from tests.torch_kernels import _plain as torch_kernel_plain
    s = r.cache.allocate_slot()
    r.step([SequenceInput(s, toks, 0, [18])])
    assert len(seen) == want.shape[0] == 8
    for i, (got, ref) in enumerate(zip(seen, want)):
        torch.testing.assert_close(got, ref, atol=2e-4, rtol=1e-4, msg=lambda m, i=i: f"layer run {i}: {m}")


def generate_plain(cfg, w, prompt, new):
    ids = list(prompt)
    for _ in range(new):
        ids.append(int(torch.argmax(pz.forward(cfg, w, ids)[-1])))
    return ids[len(prompt):]


def test_greedy_generation_through_the_entry_point_on_cpu(model_dirs, torch_ops):
    d = model_dirs["z3"]
    cfg, w = pz.read_model_dir(d, torch.float32)
    prompts = zu.requests(cfg["vocab"], [3, 20, 9], 7)
    want = [generate_plain(cfg, w, p, 10) for p in prompts]
    eng = Engine(EngineConfig(model_path=str(d), dtype="float32", device="cpu", kv_pool_tokens=96, page_size=8,
                              max_reqs=2, max_seq_len=64, max_prefill_tokens=12, cuda_graphs=False,
                              async_scheduling=False))
    outs = eng.generate(prompts, SamplingParams(max_new_tokens=10, ignore_eos=True))
    assert [o.token_ids for o in outs] == want
    eng.cache.check_invariants()


def test_the_command_line_writes_a_model_folder_the_registry_reads_back(tmp_path):
    from deterministic_inference_b200.__main__ import main
    from deterministic_inference_b200.config import preset
    cfg = preset("zatirax_tiny")
    assert isinstance(cfg, ZatiraxConfig)
    out = tmp_path / "model"
    assert main(["random", "--preset", "zatirax_tiny", "--seed", "3", "--out", str(out)]) == 0
    back = config_from_dir(out)
    assert back.to_dict() == cfg.to_dict()
    model = build_model(back, torch.float32, "cpu")
    load_weights(out, model.tensor_specs(), model.plan, torch.float32, "cpu")
