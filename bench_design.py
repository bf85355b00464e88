"""``bench.py --design mapuvik`` / ``gagotar`` / ``semadra`` / ``rizitar``: prefill and decode
throughput of the design at sizes that resemble a real model's layers, beside GPT-2 of the same
width, heads, feed-forward and number of layers (Gagotar also beside Mapuvik, the design whose
kernels are closest to its own; Semadra beside Gagotar, whose experts and attention, and
Mapuvik, whose latent attention are the like kernels; Rizitar beside Semadra, whose windowed
attention, norms behind the sublayers, experts and token input, and Gagotar, whose scan over a
matrix state are the like kernels), on one B200 with random bf16 weights.

For each size and model: one prompt step of 2,048 tokens (two prompts of 1,024) and one decode
step of 8 requests at context 1,025, each timed on the device as a CUDA-graph replay of the
model's forward (no host time between kernels), and per kernel class: in the prompt step the
class's own kernels between CUDA events (``ops.timed``), in the decode step the step with and
without the class (``ops.leaving_out``). A class's ``frac`` is its arithmetic over the measured
bf16 peak (products and attention of the prompt step) or its bytes over the measured copy
bandwidth (everything else), so that like kernels of the two models can be set side by side.
``generate`` is the decode step through ``LLM.generate`` (scheduler, sampling and host time
included, CUDA graphs on). One JSON line.
"""

from __future__ import annotations

import json
import tempfile
from pathlib import Path

PROMPTS, LENGTH, BATCH = 2, 1024, 8


def mapuvik_config(width: int, heads: int, ff: int, repeats: int, vocab: int) -> dict:
    head = width // heads
    latent = {"type": "latent_attention", "mixer": {
        "heads": heads, "dim": head, "rot_dim": head // 2, "vdim": head,
        "kv_rank": 256 - head // 2,
        "scale": (head + head // 2) ** -0.5, "mask": {"size": LENGTH},
        "rot": {"base": 10000.0, "dims": head // 2}}}
    mamba = {"type": "mamba2", "mixer": {"heads": 2 * width // 64, "vdim": 64, "state": 128,
                                         "groups": 1, "conv": 4, "norm_groups": 1}}
    memory_heads = max(1, width // 256)
    mlstm = {"type": "mlstm", "mixer": {"heads": memory_heads, "dim": width // memory_heads,
                                        "vdim": width // memory_heads, "gate_cap": 15.0}}
    mlp = {"kind": "dense", "ff": ff}
    layers = [{**kind, "mlp": mlp} for _ in range(repeats) for kind in (latent, mamba, mlstm)]
    return {"architecture": "Mapuvik", "vocab": vocab, "width": width, "norm": {"eps": 1e-5},
            "layers": layers}


#: Gagotar at the bench's sizes: blocks of 384 positions (a prompt of 1,024 holds two and
#: two thirds of one, and the decode step at context 1,025 sees 257 keys); experts of a
#: quarter of the dense feed-forward's width, two of sixteen per row
GAGOTAR_CHUNK, GAGOTAR_EXPERTS, GAGOTAR_TOP = 384, 16, 2


def gagotar_config(width: int, heads: int, ff: int, layers: int, vocab: int) -> dict:
    head = width // heads
    left = {"heads": heads, "kv_heads": heads // 4, "dim": head, "vdim": head,
            "scale": head ** -0.5, "mask": {"size": GAGOTAR_CHUNK},
            "rot": {"base": 500000.0, "dims": head,
                    "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 8192}}}
    memory_heads = max(1, width // 256)
    right = {"heads": memory_heads, "dim": 128, "vdim": width // memory_heads, "tau": 16.0,
             "rank": 16}
    mlp = {"kind": "moe", "expert": {"ff": ff // 4, "limit": 7.0},
           "router": {"experts": GAGOTAR_EXPERTS, "top": GAGOTAR_TOP}}
    entry = {"type": "parallel", "mixer": {"left": left, "right": right}, "mlp": mlp}
    return {"architecture": "Gagotar", "vocab": vocab, "width": width, "norm": {"eps": 1e-5},
            "layers": [entry for _ in range(layers)]}


#: Semadra at the bench's sizes: windows of 512 positions (a prompt of 1,024 passes over
#: them, the decode step at context 1,025 sees 512 keys, the gated attention 64 kept ones
#: more); latents of 256 entries (a row size the engine's own attention kernels take); a dense
#: first layer, then experts as in Gagotar's configuration with a shared one beside them
SEMADRA_WINDOW, SEMADRA_KEEP, SEMADRA_EXPERTS, SEMADRA_TOP = 512, 64, 16, 2


def semadra_config(width: int, heads: int, ff: int, repeats: int, vocab: int) -> dict:
    head = width // heads
    latent = {"heads": heads, "dim": head, "vdim": head, "kv_rank": 256, "q_rank": width // 2,
              "scale": head ** -0.5, "mask": {"size": SEMADRA_WINDOW}}
    attention = {"heads": heads, "kv_heads": heads // 4, "dim": head, "vdim": head,
                 "scale": head ** -0.5,
                 "mask": {"size": SEMADRA_WINDOW, "keep_first": SEMADRA_KEEP}}
    moe = {"kind": "moe", "expert": {"ff": ff // 4}, "shared": {"ff": ff // 4},
           "router": {"experts": SEMADRA_EXPERTS, "top": SEMADRA_TOP, "scale": 2.5,
                      "groups": {"count": 4, "keep": 2}}}
    layers = []
    for repeat in range(repeats):
        at = 3 * repeat
        layers += [
            {"type": "latent_attention", "mixer": dict(latent),
             "mlp": moe if repeat else {"kind": "dense", "ff": ff}},
            {"type": "latent_attention", "mixer": {**latent, "kv_from": at}, "mlp": moe},
            {"type": "attention", "mixer": attention, "mlp": moe}]
    return {"architecture": "Semadra", "vocab": vocab, "width": width, "norm": {"eps": 1e-5},
            "embedding": {"scale": width ** 0.5}, "residual_mult": 0.5,
            "token_side": {"dim": 64}, "layers": layers}


#: Rizitar at the bench's sizes: windows of 512 positions behind which blocks of 16 are pooled
#: (the decode step at context 1,025 sees 512 keys and 32 pooled rows), heads wholly rotated
#: with blended frequencies; delta layers with heads of 64 channels; a dense feed-forward in
#: the first layer of three, experts as in Gagotar's configuration in the other two
RIZITAR_WINDOW, RIZITAR_POOL, RIZITAR_EXPERTS, RIZITAR_TOP = 512, 16, 16, 2


def rizitar_config(width: int, heads: int, ff: int, repeats: int, vocab: int) -> dict:
    head = width // heads
    attention = {"heads": heads, "kv_heads": heads // 4, "dim": head, "vdim": head,
                 "scale": head ** -0.5, "mask": {"size": RIZITAR_WINDOW, "pool": RIZITAR_POOL},
                 "rot": {"base": 500000.0, "dims": head,
                         "scaling": {"factor": 4.0, "original": 8192, "fast": 16.0,
                                     "slow": 1.0}}}
    memory = {"heads": width // 64, "dim": 64, "decay_rank": 64}
    moe = {"kind": "moe", "expert": {"ff": ff // 4},
           "router": {"experts": RIZITAR_EXPERTS, "top": RIZITAR_TOP}}
    layers = []
    for _ in range(repeats):
        layers += [
            {"type": "attention", "mixer": attention, "mlp": {"kind": "dense", "ff": ff}},
            {"type": "attention", "mixer": attention, "mlp": moe},
            {"type": "general_delta", "mixer": memory, "mlp": moe}]
    return {"architecture": "Rizitar", "vocab": vocab, "width": width, "norm": {"eps": 1e-5},
            "embedding": {"scale": width ** 0.5}, "token_side": {"dim": 64}, "layers": layers}


def gpt2_config(width: int, heads: int, ff: int, layers: int, vocab: int) -> dict:
    return {"architectures": ["GPT2LMHeadModel"], "n_layer": layers, "n_embd": width,
            "n_head": heads, "n_inner": ff, "vocab_size": vocab, "n_positions": 2 * LENGTH,
            "layer_norm_epsilon": 1e-5, "activation_function": "gelu_new",
            "scale_attn_by_inverse_layer_idx": False, "tie_word_embeddings": True}


def _core(config: dict):
    import torch

    from ayaka_b200.config.engine import EngineConfig
    from ayaka_b200.engine.core import EngineCore
    from ayaka_b200.weights.random_init import random_state

    state = random_state(config, 0, None, "bfloat16")
    with tempfile.TemporaryDirectory() as folder:
        (Path(folder) / "config.json").write_text(json.dumps(config))
        core = EngineCore.from_config(
            EngineConfig(model=folder, dtype="bfloat16", device="cuda:0", block_size=16,
                         num_blocks=BATCH * (LENGTH + 64) // 16 + 1, max_running=BATCH,
                         max_tokens_per_step=PROMPTS * LENGTH, max_context=LENGTH + 64),
            tensors=state)
    del state
    torch.cuda.synchronize()
    return core


def _tokens(vocab: int, count: int, seed: int) -> list[int]:
    import torch

    return torch.randint(0, vocab, (count,), generator=torch.Generator().manual_seed(seed)).tolist()


def _class_work(config: dict, rows: int, keys_per_row: float, decode: bool,
                wanted: int) -> dict[str, dict]:
    """Per kernel class of a step: FLOPs and bytes summed over the layers. ``keys_per_row``:
    mean number of keys a row attends; ``wanted``: rows that reach the head."""
    work: dict[str, dict] = {}

    def add(name: str, flops: float, nbytes: float) -> None:
        entry = work.setdefault(name, {"flops": 0.0, "bytes": 0.0})
        entry["flops"] += flops
        entry["bytes"] += nbytes

    def product(n: int, k: int, out_bytes: int = 2, m: int = rows) -> None:
        add(f"linear:{n}x{k}", 2.0 * m * n * k, n * k * 2 + m * (k * 2 + n * out_bytes))

    if "n_embd" in config:
        d, f, h = config["n_embd"], config["n_inner"], config["n_head"]
        for _ in range(config["n_layer"]):
            product(3 * d, d)
            product(d, d, 4)
            product(f, d)
            product(d, f, 4)
            add("attention", 4.0 * rows * keys_per_row * d, rows * keys_per_row * 2 * d * 2 / (
                1 if decode else LENGTH / 8))
            add("layer_norm", 0.0, 2 * rows * d * 6)
        product(config["vocab_size"], d, 4, wanted)
        return work
    width = config["width"]
    if config["architecture"] == "Gagotar":
        for layer in config["layers"]:
            a, r, mlp = layer["mixer"]["left"], layer["mixer"]["right"], layer["mlp"]
            H, G, dim, vdim = a["heads"], a["kv_heads"], a["dim"], a["vdim"]
            chunk = a["mask"]["size"]
            # keys a row sees: half a block on average in a prompt; in a decode step the
            # place of the context's last position in its block
            keys = (int(keys_per_row) - 1) % chunk + 1 if decode else \
                sum(p % chunk + 1 for p in range(LENGTH)) / LENGTH
            add("rms_norm", 0.0, 2 * rows * width * 6)
            product(H * dim + G * dim + G * vdim + H, width, 4)
            product(width, H * vdim, 4)
            add("talking_prepare", 2.0 * rows * H * H * dim,
                rows * ((H * dim + G * (dim + vdim)) * 4 + (H * G * dim + G * (dim + vdim)) * 2))
            add("talking_attention", 2.0 * rows * keys * H * (dim + vdim + H),
                rows * keys * G * (dim + vdim) * 2 / (1 if decode else chunk / 8)
                + rows * H * (G * dim + vdim) * 2)
            Hr, N, P = r["heads"], r["dim"], r["vdim"]
            product(2 * Hr * N + 2 * Hr * P, width, 4)
            product(r["rank"], width)
            product(Hr * N, r["rank"], 4)
            product(width, Hr * P, 4)
            add("gla_scan", 6.0 * rows * Hr * N * P,
                rows * (3 * Hr * N + 2 * Hr * P) * 4 + (2 * Hr * N * P * 4) * (
                    rows if decode else 2))
            add("rms_norm", 0.0, rows * Hr * P * 10)
            add("norm_sum", 0.0, rows * width * 16)
            E, top, f = mlp["router"]["experts"], mlp["router"]["top"], mlp["expert"]["ff"]
            product(E, width, 4)
            add("moe_route", 0.0, rows * (E + 2 * top) * 4)
            add("moe_experts", 2.0 * rows * top * 3 * f * width,
                min(E, rows * top) * 3 * f * width * 2 + rows * top * (width * 6 + f * 4))
            add("moe_join", 0.0, rows * width * (4 * top + 8))
        product(config["vocab"], width, 4, wanted)
        return work
    if config["architecture"] == "Rizitar":
        side = (config.get("token_side") or {}).get("dim", 0)
        # (only the first layer launches the norm in front of its mixer: every other norm in
        # front of a sublayer leaves the launch that last updated the stream, `norm_add`,
        # which then writes one more row in the compute type)
        add("rms_norm", 0.0, rows * width * 6)
        for layer in config["layers"]:
            m, mlp = layer["mixer"], layer["mlp"]
            if layer["type"] == "attention":
                H, G, dim = m["heads"], m.get("kv_heads", m["heads"]), m["dim"]
                window = (m.get("mask") or {}).get("size", 0)
                pool = (m.get("mask") or {}).get("pool", 0)

                def seen(p: int) -> int:  # keys and pooled rows the row at position p attends
                    if not window or p < window:
                        return p + 1
                    return window + ((p - window + 1) // pool if pool else 0)

                keys = seen(int(keys_per_row) - 1) if decode else \
                    sum(seen(p) for p in range(LENGTH)) / LENGTH
                reuse = 1 if decode else 64 / 8  # a tile of 64 rows shares its keys
                product(H * dim + G * dim, width, 4)
                add("pooled_prepare", 0.0, rows * (H * dim + G * dim) * 4
                    + rows * (H * dim + 2 * G * dim) * 2)
                if pool:
                    add("pooled_blocks", 0.0, rows * G * 2 * dim * 2 * (1 + 1 / pool))
                add("pooled_attention", 4.0 * rows * keys * H * dim,
                    rows * keys * G * 2 * dim * 2 / reuse + rows * H * dim * 4)
                product(width, H * dim, 4)
            else:
                H, N, rank = m["heads"], m["dim"], m["decay_rank"]
                product(5 * H * N + rank, width, 4)
                add("unary_rows", 0.0, rows * rank * 6)
                product(H * N, rank, 4)
                add("delta_scan", 8.0 * rows * H * N * N,
                    rows * 6 * H * N * 4 + (2 * H * N * N * 4) * (rows if decode else PROMPTS))
                add("rms_norm", 0.0, rows * H * N * 10)
                product(width, H * N, 4)
            add("norm_add", 0.0, rows * width * 16)
            if mlp is not None:
                if mlp["kind"] == "dense":
                    product(mlp["ff"], width, 4)
                    add("unary_rows", 0.0, rows * mlp["ff"] * 6)
                    product(width, mlp["ff"], 4)
                else:
                    E, top, f = mlp["router"]["experts"], mlp["router"]["top"], mlp["expert"]["ff"]
                    product(E, width, 4)
                    add("moe_route", 0.0, rows * (E + 2 * top) * 4)
                    add("moe_experts", 2.0 * rows * top * 2 * f * width,
                        min(E, rows * top) * 2 * f * width * 2 + rows * top * (width * 6 + f * 4))
                    add("moe_join", 0.0, rows * width * (4 * top + 4))
                add("norm_add", 0.0, rows * width * 16)
            if side:
                product(side, width, 4)
                add("gated_unit", 0.0, rows * side * 8)
                product(width, side, 4)
                add("norm_add", 0.0, rows * width * 16)
        add("rms_norm", 0.0, wanted * width * 6)
        product(config["vocab"], width, 4, wanted)
        return work
    if config["architecture"] == "Semadra":
        side = (config.get("token_side") or {}).get("dim", 0)
        add("cast_rows", 0.0, rows * width * 6)

        def gated(inner: int) -> None:  # act(gate) * up between two products
            product(2 * inner, width, 4)
            add("gated_unit", 0.0, rows * inner * 10)
            product(width, inner, 4)

        for layer in config["layers"]:
            m, mlp = layer["mixer"], layer["mlp"]
            H, dim, vdim = m["heads"], m["dim"], m["vdim"]
            window = (m.get("mask") or {}).get("size", 0)
            keep = (m.get("mask") or {}).get("keep_first", 0)

            def seen(p: int) -> int:  # keys the row at position p attends
                if not window or p < window:
                    return p + 1
                return window + min(keep, p + 1 - window)

            keys = seen(int(keys_per_row) - 1) if decode else \
                sum(seen(p) for p in range(LENGTH)) / LENGTH
            reuse = 1 if decode else 64 / 8  # a tile of 64 rows shares its keys
            if layer["type"] == "attention":
                G = m.get("kv_heads", H)
                product(H * dim + G * (dim + vdim) + H * vdim, width, 4)
                add("gated_attention_prepare", 0.0,
                    rows * (H * dim + G * (dim + vdim)) * 6)
                add("gated_attention", 2.0 * rows * keys * H * (dim + vdim),
                    rows * keys * G * (dim + vdim) * 2 / reuse + rows * H * (dim + 5 * vdim))
            else:
                rank, q_rank = m["kv_rank"], m["q_rank"]
                own = 0 if "kv_from" in m else rank
                product(q_rank + own, width, 4)
                add("rms_norm", 0.0, rows * q_rank * 6)
                product(H * dim, q_rank, 4)
                add("latent_prepare", 0.0, rows * (H * dim * 6 + own * 6))
                add("head_linear", 2.0 * rows * H * rank * (dim + vdim),
                    H * rank * (dim + vdim) * 2 + rows * H * (dim + vdim + 2 * rank) * 2)
                add("latent_attention", 4.0 * rows * keys * H * rank,
                    rows * keys * rank * 2 / reuse)
            product(width, H * vdim, 4)
            add("norm_add", 0.0, rows * width * 14)
            if mlp is not None:
                if mlp["kind"] == "dense":
                    gated(mlp["ff"])
                else:
                    E, top, f = mlp["router"]["experts"], mlp["router"]["top"], mlp["expert"]["ff"]
                    product(E, width, 4)
                    add("moe_route_scored", 0.0, rows * (E + 2 * top) * 4)
                    add("moe_experts", 2.0 * rows * top * 3 * f * width,
                        min(E, rows * top) * 3 * f * width * 2 + rows * top * (width * 6 + f * 4))
                    add("moe_join", 0.0, rows * width * (4 * top + 8))
                    if mlp.get("shared"):
                        gated(mlp["shared"]["ff"])
                add("norm_add", 0.0, rows * width * 14)
            if side:
                product(side, width, 4)
                add("gated_unit", 0.0, rows * side * 8)
                product(width, side, 4)
                add("norm_add", 0.0, rows * width * 14)
        add("rms_norm", 0.0, wanted * width * 6)
        product(config["vocab"], width, 4, wanted)
        return work
    for layer in config["layers"]:
        m = layer["mixer"]
        if layer["mlp"]:
            product(layer["mlp"]["ff"], width)
            product(width, layer["mlp"]["ff"], 4)
        add("rms_norm", 0.0, rows * width * 6)
        if layer["type"] == "latent_attention":
            H, dim, rot, vdim, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
            product(H * (dim + rot) + rank + rot + H * vdim, width, 4)
            product(width, H * vdim, 4)
            add("latent_prepare", 0.0, rows * (H * (dim + rot) * 6 + (rank + rot) * 6))
            add("head_linear", 2.0 * rows * H * rank * (dim + vdim),
                H * rank * (dim + vdim) * 2 + rows * H * (dim + vdim + 2 * rank) * 2)
            # every head scores rank + rot entries and sums rank entries of each key row; a
            # decode step must read each request's rows once, whatever the number of heads
            add("latent_attention", 2.0 * rows * keys_per_row * H * (2 * rank + rot),
                rows * keys_per_row * (rank + rot) * 2 / (1 if decode else LENGTH / 8))
        elif layer["type"] == "mamba2":
            H, P, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
            inner, channels = H * P, H * P + 2 * G * N
            product(2 * inner + 2 * G * N + H, width, 4)
            product(width, inner, 4)
            add("causal_conv_silu", 2.0 * rows * channels * m["conv"], rows * channels * 8)
            add("mamba2_scan", 6.0 * rows * H * N * P,
                rows * (channels + H + inner) * 4 + (2 * H * N * P * 4) * (rows if decode else 2))
            add("rms_norm", 0.0, rows * inner * 10)
        else:
            H, dim, P = m["heads"], m["dim"], m["vdim"]
            product(2 * H * dim + 2 * H * P + 2 * H, width, 4)
            product(width, H * P, 4)
            add("mlstm_scan", 6.0 * rows * H * dim * P,
                rows * (2 * H * dim + 2 * H * P) * 4 + (2 * H * dim * P * 4) * (
                    rows if decode else 2))
            add("rms_norm", 0.0, rows * H * P * 10)
    product(config["vocab"], width, 4, wanted)
    return work


def _generate(core, vocab: int) -> dict:
    """Decode throughput through the Python entry point and the scheduler (host time
    included): 8 prompts of 128 tokens, (time of 65 new tokens - time of 1) / 64, greedy,
    CUDA graphs on."""
    import time

    import torch

    from ayaka_b200.config.engine import EngineConfig
    from ayaka_b200.engine.llm import LLM
    from ayaka_b200.sampling.params import SamplingParams

    config = EngineConfig(model=".", dtype="bfloat16", device="cuda:0", block_size=16,
                          num_blocks=core.manager.pools[0].num_pages, max_running=BATCH,
                          max_tokens_per_step=PROMPTS * LENGTH, max_context=LENGTH + 64,
                          cuda_graph=True)
    llm = LLM(core, config)
    prompts = [tuple(_tokens(vocab, 128, 40 + i)) for i in range(BATCH)]
    times = {}
    for new in (1, 65, 1, 65):  # (the first pair warms up and captures the graphs)
        torch.cuda.synchronize()
        start = time.perf_counter()
        llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=new, ignore_eos=True))
        torch.cuda.synchronize()
        times[new] = time.perf_counter() - start
    llm.close()
    step = (times[65] - times[1]) / 64
    return {"ms_per_step": round(step * 1000, 4), "tok_s": round(BATCH / step, 1),
            "graph_replays": 0 if llm.graphs is None else llm.graphs.replays}


def _measure(config: dict, peak: dict) -> dict:
    import torch

    from bench import _timed_graph
    from ayaka_b200.engine.runner import StepEntry
    from ayaka_b200.kernels import ops

    core = _core(config)
    vocab = config.get("vocab") or config["vocab_size"]
    model, runner, manager = core.model, core.runner, core.manager
    tflops, gbs = peak["bf16_tflops"] * 1e12, peak["hbm_gbs"] * 1e9
    out: dict[str, object] = {}

    def forward_of(entries):  # the step's context, as the engine prepares it
        for entry in entries:
            assert manager.allocate(entry.request_id, len(entry.tokens))
        step, want_rows, num_want = runner.prepare(entries)
        return lambda: model.forward(step, runner.caches, want_rows, num_want)

    def commit(entries) -> None:
        for entry in entries:
            manager.commit(entry.request_id, len(entry.tokens))

    def classes(body, work, decode: bool, step_ms: float) -> dict:
        found: dict[str, dict] = {}
        if decode:
            for name in work:
                # (attention over latent rows runs in the engine's own attention kernels
                # where the row's size is one they take)
                left = {"attention": ("attention_decode",),
                        "latent_attention": ("latent_attention", "latent_decode",
                                             "attention_decode")}.get(
                            name, (name,))
                with ops.leaving_out(*left):
                    without = _timed_graph(body, 5)
                found[name] = {"us": round(max(step_ms - without, 0.0) * 1000, 1)}
        else:
            filler = torch.empty(64 << 20, device="cuda")
            for _ in range(2):
                with ops.timed() as record:
                    for _ in range(60):  # (a step of 300 launches takes the host 3 ms)
                        filler.zero_()  # the device is busy while the host queues the step
                    body()
                torch.cuda.synchronize()
            for klass, pairs in record.items():
                name = klass
                if klass == "attention_prefill":
                    name = "pooled_attention" if "pooled_attention" in work else (
                        "latent_attention" if "latent_attention" in work else "attention")
                elif klass == "latent_decode":
                    name = "latent_attention"
                if name in work:
                    us = sum(start.elapsed_time(stop) for start, stop in pairs) * 1000
                    found.setdefault(name, {"us": 0.0})["us"] += us
            for name in found:
                found[name]["us"] = round(found[name]["us"], 1)
        for name, entry in found.items():
            seconds = max(entry["us"], 1e-3) * 1e-6
            by_flops = work[name]["flops"] / seconds / tflops
            by_bytes = work[name]["bytes"] / seconds / gbs
            tensor = not decode and "prepare" not in name and (
                name.startswith("linear") or "attention" in name
                or name in ("head_linear", "moe_experts"))
            entry["frac"] = round(by_flops if tensor else by_bytes, 4)
            entry["of"] = "bf16_tflops" if tensor else "hbm_gbs"
        return found

    # ---- the prompt step
    prompts = [StepEntry(f"p{i}", _tokens(vocab, LENGTH, i), (LENGTH - 1,))
               for i in range(PROMPTS)]
    native = ops.NATIVE_STEP
    body = forward_of(prompts)
    ms = _timed_graph(body, 5)
    ops.NATIVE_STEP = False  # one Python call per kernel: where a class can be timed
    try:
        rows = PROMPTS * LENGTH
        out["prefill"] = {"ms": round(ms, 3), "tok_s": round(rows * 1000.0 / ms, 1),
                          "classes": classes(body, _class_work(config, rows, (LENGTH + 1) / 2,
                                                               False, PROMPTS), False, ms)}
        commit(prompts)
        for i in range(PROMPTS, BATCH):  # the other requests of the decode batch
            extra = [StepEntry(f"p{i}", _tokens(vocab, LENGTH, i), ())]
            core.step(extra)
        # ---- the decode step
        ops.NATIVE_STEP = native
        decodes = [StepEntry(f"p{i}", [7 + i], (0,)) for i in range(BATCH)]
        body = forward_of(decodes)
        ms = _timed_graph(body, 10)
        ops.NATIVE_STEP = False
        body_classes = forward_of(decodes)
        out["decode"] = {"ms": round(ms, 4), "tok_s": round(BATCH * 1000.0 / ms, 1),
                         "batch": BATCH, "context": LENGTH + 1,
                         "classes": classes(body_classes, _class_work(
                             config, BATCH, LENGTH + 1, True, BATCH), True,
                             _timed_graph(body_classes, 10))}
    finally:
        ops.NATIVE_STEP = native
    runner.check_device_flags()
    for i in range(BATCH):
        core.release(f"p{i}")
    out["generate"] = _generate(core, vocab)
    del core
    torch.cuda.empty_cache()
    return out


def run(sizes: str | None = None, design: str = "mapuvik") -> dict:
    from bench import peaks

    peak, source = peaks()
    table = {"1024": (1024, 16, 4096, 2), "2048": (2048, 16, 8192, 2)}
    picked = [s for s in (sizes.split(",") if sizes else table) if s in table]
    results = {}
    for name in picked:
        width, heads, ff, repeats = table[name]
        results[name] = {"layers": 3 * repeats, "width": width, "heads": heads, "ff": ff}
        if design == "rizitar":
            results[name]["rizitar"] = _measure(
                rizitar_config(width, heads, ff, repeats, 32000), peak)
        if design in ("semadra", "rizitar"):
            results[name]["semadra"] = _measure(
                semadra_config(width, heads, ff, repeats, 32000), peak)
        if design in ("gagotar", "semadra", "rizitar"):
            results[name]["gagotar"] = _measure(
                gagotar_config(width, heads, ff, 3 * repeats, 32000), peak)
        if design != "rizitar":
            results[name]["mapuvik"] = _measure(
                mapuvik_config(width, heads, ff, repeats, 32000), peak)
        results[name]["gpt2"] = _measure(gpt2_config(width, heads, ff, 3 * repeats, 32000), peak)
    title = {"rizitar": "Rizitar beside Semadra, Gagotar and GPT-2",
             "gagotar": "Gagotar beside Mapuvik and GPT-2",
             "semadra": "Semadra beside Gagotar, Mapuvik and GPT-2"}.get(
                 design, "Mapuvik beside GPT-2")
    return {"metric": f"{title} of equal size: one 2,048-token prompt step and one "
                      "decode step of 8 requests at context 1,025 (bf16, random weights)",
            "peaks": {**{k: peak[k] for k in ("hbm_gbs", "bf16_tflops")}, "source": source},
            "timing": "CUDA-graph replay of the model's forward, device time, best of 5 / 10",
            "sizes": results}
