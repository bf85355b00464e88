"""Semadra on the CPU: configuration, model description, checkpoint rules, the cache plan of
layers that share latents and of windows that keep first tokens, and the plain
implementation's own consistency (each mechanism against a formula written out by hand)."""

from __future__ import annotations

import copy
import math

import pytest
import torch

import plain_semadra as plain
from semadra_cases import LOUD, TINY_A, TINY_B, TINY_C, TINY_D
from ayaka_b200.cache.manager import CacheManager
from ayaka_b200.cache.storage import plan_cache
from ayaka_b200.config.semadra import SemadraConfig
from ayaka_b200.errors import AyakaError, ModelLoadError
from ayaka_b200.models import build_model
from ayaka_b200.models.registry import architecture_of
from ayaka_b200.parts.base import CacheNeed
from ayaka_b200.weights.loader import TensorSource, load_into
from ayaka_b200.weights.random_init import random_state


def test_the_configuration_reads_back_as_written():
    for raw in (TINY_A, TINY_B, TINY_C, TINY_D):
        config = SemadraConfig.from_json_dict(raw)
        assert SemadraConfig.from_json_dict(config.to_json_dict()) == config
        assert [layer.kind for layer in config.layers] == [e["type"] for e in raw["layers"]]
    a = SemadraConfig.from_json_dict(TINY_A)
    assert (a.embedding_scale, a.residual_mult, a.side_dim) == (4.0, 0.4, 6)
    assert [layer.kv_from for layer in a.layers] == [None, None, 0, None]
    assert (a.layers[1].kv_heads, a.layers[1].window, a.layers[1].keep_first) == (2, 9, 13)
    assert a.layers[1].mlp.groups == 3 and a.layers[1].mlp.keep == 2
    assert a.layers[3].mlp.groups == 1 and a.layers[3].mlp.shared_ff == 0
    b = SemadraConfig.from_json_dict(TINY_B)
    # what a file may leave out: factors of one, no side input, no window, no kept tokens
    assert (b.embedding_scale, b.residual_mult, b.side_dim) == (1.0, 1.0, 0)
    assert b.layers[2].window == 0 and b.layers[2].keep_first == 0 and b.layers[1].mlp is None


@pytest.mark.parametrize("change, text", [
    (lambda c: c.pop("vocab"), "vocab"),
    (lambda c: c["norm"].pop("eps"), "norm.eps"),
    (lambda c: c["layers"][0]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda c: c["layers"][1]["mixer"].pop("scale"), "scale"),
    (lambda c: c["layers"][1].update(type="mamba2"), "not a mixer"),
    (lambda c: c["layers"][0]["mlp"].update(kind="glu"), "dense, moe"),
    (lambda c: c["layers"][2]["mixer"].update(kv_from=2), "earlier"),
    (lambda c: c["layers"][2]["mixer"].update(kv_from=1), "earlier latent"),
    (lambda c: c["layers"][2]["mixer"].update(kv_rank=16), "same kv_rank"),
    (lambda c: c["layers"][1]["mixer"].update(kv_heads=3), "divide heads"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=5), "kept groups"),
    (lambda c: c["layers"][1]["mlp"]["router"]["groups"].update(count=4), "divide experts"),
    (lambda c: c["layers"][3]["mlp"]["expert"].update(ff=0), "at least 1"),
    (lambda c: c.update(token_side={"dim": 0}), "at least 1"),
])
def test_a_configuration_that_lacks_or_twists_something_is_refused(change, text):
    raw = copy.deepcopy(TINY_A)
    change(raw)
    with pytest.raises(AyakaError, match=text):
        SemadraConfig.from_json_dict(raw)


def test_the_cache_plan_shares_latents_and_keeps_first_pages():
    model, _, _ = build_model(TINY_A, "float32", "cpu")
    spec = model.spec
    assert [run.reads_cache_of for run in spec.order] == [None, None, 0, None]
    plan = plan_cache(spec.order, model.needs())
    assert plan.run_writes == (True, True, False, True)
    assert plan.run_slot[2] == plan.run_slot[0] and plan.run_group[2] == plan.run_group[0]
    shared = plan.groups[plan.run_group[0]]
    # the owner looks 11 back, its reader 37: the slot keeps what the reader still sees
    assert shared.values is False and shared.head_dim == 32 and shared.window == 37
    first = plan.groups[plan.run_group[1]]
    assert (first.num_kv_heads, first.head_dim, first.value_head_dim) == (2, 16, 8)
    assert (first.window, first.keep_first) == (9, 13)
    # an attention without a window keeps everything and has no use for kept tokens
    model_b, _, _ = build_model(TINY_B, "float32", "cpu")
    plan_b = plan_cache(model_b.spec.order, model_b.needs())
    free = plan_b.groups[plan_b.run_group[2]]
    assert free.window == 0 and free.keep_first == 0


def test_the_manager_never_gives_back_the_pages_of_kept_tokens():
    """Window 6, 5 kept tokens, pages of 4: pages 0 and 1 stay whatever the length, the pages
    between them and the window go back to the pool and come round again."""
    need = CacheNeed(1, 8, 6, keep_first=5)
    manager = CacheManager([need], [9], 4, 1, 40)
    assert manager.allocate("r", 3)
    manager.commit("r", 3)
    held = []
    for _ in range(120):
        assert manager.allocate("r", 1)
        manager.commit("r", 1)
        manager.check_integrity()
        table = manager.tables[0][manager.row("r")]
        held.append(int((table != 0).sum()))
        assert int(table[0]) != 0 and (manager.committed("r") <= 4 or int(table[1]) != 0)
    # at most the two kept pages and the three a window of 6 can touch: 123 tokens went
    # through a pool of 8 pages
    assert max(held) <= 5
    assert manager.num_free_pages(0) >= 8 - 5
    manager.free("r")
    manager.check_integrity()
    assert manager.num_free_pages(0) == 8


def test_random_tensors_fill_the_model_exactly():
    for raw in (TINY_A, TINY_B, TINY_D):
        model, architecture, config = build_model(raw, "float32", "cpu")
        state = random_state(raw, 3, LOUD)
        load_into(model, architecture.weight_rules(config), TensorSource(tensors=state))
        params = dict(model.named_params())
        if raw is TINY_A:
            fused = params["layers.1.mixer.proj.weight"].tensor
            assert torch.equal(fused, torch.cat([state[f"l1.mix.{n}"] for n in "qkvg"]))
            owner = params["layers.0.mixer.proj.weight"].tensor
            assert torch.equal(owner, torch.cat([state["l0.mix.dq"], state["l0.mix.dkv"]]))
            reader = params["layers.2.mixer.proj.weight"].tensor
            assert torch.equal(reader, state["l2.mix.dq"]) and "l2.mix.dkv" not in state
            experts = params["layers.1.feed_forward.in.weight"].tensor
            assert torch.equal(experts[2 * 48:2 * 48 + 24], state["l1.mlp.e2.gate"])
            assert torch.equal(experts[2 * 48 + 24:3 * 48], state["l1.mlp.e2.up"])
            table = params["layers.3.side.table"].tensor
            assert torch.equal(table, state["side.embed"][:, 18:24])
            assert "l2.norm2" not in state  # no feed-forward, no second norm
        del state["final.norm"]
        with pytest.raises(ModelLoadError, match="missing"):
            load_into(model, architecture.weight_rules(config), TensorSource(tensors=state))
    assert architecture_of({"architecture": "Semadra"}).name == "Semadra"


# ---- the plain implementation against formulas written out by hand ----------------------------
def test_the_plain_mask_at_its_edges():
    mask = plain.visible(30, 7, 3)
    assert mask[20, 14] and not mask[20, 13]          # seven keys: itself and six before
    assert mask[20, 2] and not mask[20, 3]            # the first three stay
    assert mask[5, 0] and not mask[5, 6]              # nothing later
    assert bool(plain.visible(30, 1)[9].sum() == 1)   # a window of one: itself
    assert bool(plain.visible(12, 12).tril().equal(plain.visible(12, 12)))


def test_the_plain_choice_of_experts_by_hand():
    # 6 experts in 3 groups of 2, the best 2 groups, 2 experts
    s = torch.tensor([[0.9, 0.1, 0.6, 0.5, 0.8, 0.0]], dtype=torch.float64)
    # group sums 1.0, 1.1, 0.8: groups 1 and 0 stay although expert 4 is second largest
    assert plain.expert_choice(s, 2, 3, 2).tolist() == [[0, 2]]
    assert plain.expert_choice(s, 2, 1, 1).tolist() == [[0, 4]]
    # groups of three: only the two largest of a group count towards its score
    s = torch.tensor([[0.5, 0.5, 0.5, 0.7, 0.6, 0.0]], dtype=torch.float64)
    assert plain.expert_choice(s, 1, 2, 1).tolist() == [[3]]
    # groups of one: a group's score is its expert's
    s = torch.tensor([[0.2, 0.9, 0.4, 0.8]], dtype=torch.float64)
    assert plain.expert_choice(s, 2, 4, 3).tolist() == [[1, 3]]
    margin = plain.choice_margin(s, 2, 4, 3)
    assert math.isclose(float(margin), 0.2, rel_tol=1e-12)  # groups: 0.4 against 0.2


def test_the_plain_model_is_causal_and_its_windows_drop_what_they_should():
    state = plain.cast_state(random_state(TINY_A, 5, LOUD), torch.float64)
    tokens = torch.randint(0, TINY_A["vocab"], (60,), generator=torch.Generator().manual_seed(1))
    whole = plain.logits(state, TINY_A, tokens)
    for cut in (1, 2, 9, 23):
        assert torch.allclose(plain.logits(state, TINY_A, tokens[:cut]), whole[:cut],
                              rtol=1e-10, atol=1e-10)
    h = torch.randn(40, 64, dtype=torch.float64, generator=torch.Generator().manual_seed(2))
    mixer = TINY_A["layers"][1]["mixer"]  # window 9, the first 13 kept
    base = plain.attention_layer(h, state, "l1.mix.", mixer, 1e-5)
    for moved_at, changes in ((39 - 9, False), (39 - 8, True), (13, False), (12, True)):
        moved = h.clone()
        moved[moved_at] += 1.0
        after = plain.attention_layer(moved, state, "l1.mix.", mixer, 1e-5)
        assert torch.equal(after[39], base[39]) != changes, moved_at
    # the reader of layer 0's latents: 37 back matters to it, not to its owner (11)
    mixer = TINY_A["layers"][2]["mixer"]
    c = plain.latent(h, state, "l0.mix.", 1e-5)
    base = plain.latent_attention_layer(h, c, state, "l2.mix.", mixer, 1e-5)
    moved = c.clone()
    moved[39 - 36] += 1.0
    assert not torch.equal(
        plain.latent_attention_layer(h, moved, state, "l2.mix.", mixer, 1e-5)[39], base[39])
    moved = c.clone()
    moved[39 - 37] += 1.0
    assert torch.equal(
        plain.latent_attention_layer(h, moved, state, "l2.mix.", mixer, 1e-5)[39], base[39])


def test_the_plain_layer_by_hand_at_one_position():
    """One token, one layer: every sum written out with Python floats."""
    raw = {"architecture": "Semadra", "vocab": 5, "width": 4, "norm": {"eps": 0.01},
           "embedding": {"scale": 3.0}, "residual_mult": 0.5, "token_side": {"dim": 2},
           "layers": [{"type": "attention", "mlp": None,
                       "mixer": {"heads": 1, "kv_heads": 1, "dim": 2, "vdim": 3, "scale": 0.7,
                                 "mask": {"size": 4, "keep_first": 1}}}]}
    state = plain.cast_state(random_state(raw, 9, LOUD), torch.float64)
    token = 3
    x = state["embed"][token] * 3.0
    # one visible key: the weights are 1, the head's output is the value row
    v = state["l0.mix.v"] @ x
    joined = v * torch.sigmoid(state["l0.mix.g"] @ x)
    y = state["l0.mix.o"] @ joined
    x1 = x + 0.5 * y / math.sqrt(float((y * y).mean()) + 0.01) * (1 + state["l0.norm1"])
    z = state["l0.side.gate"] @ x1
    g = 0.5 * z * (1 + torch.tanh(math.sqrt(2 / math.pi) * (z + 0.044715 * z ** 3)))
    s = state["l0.side.proj"] @ (g * state["side.embed"][token, :2])
    x2 = x1 + 0.5 * s / math.sqrt(float((s * s).mean()) + 0.01) * state["l0.side.norm"]
    normed = x2 / math.sqrt(float((x2 * x2).mean()) + 0.01) * (1 + state["final.norm"])
    want = state["embed"] @ normed
    got = plain.logits(state, raw, [token])[0]
    assert torch.allclose(got, want, rtol=1e-12, atol=1e-12)
