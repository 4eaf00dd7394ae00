"""The reference arm of ``bench.py``: CodeMan62/lily itself, unmodified, on the benchmark's configuration.

Nothing of ``lily_b200`` is imported here.  The reference is taken from ``baseline/_ref`` (see
``install_reference.py``), a checkpoint with the benchmark's layer sizes and seeded random weights is
written with plain ``torch`` + ``safetensors`` into a temporary folder (with a two-word tokenizer
file, because ``lily.engine.Engine`` opens a tokenizer), and the reference is driven through its own
entry point the way its own benchmark drives it (bench/bench.py:104-172 there): ``Engine`` →
``ForwardBatch.for_extend`` / ``for_decode`` → ``runner.forward``, stock Triton attention, its own
CUDA extension and cuBLAS, CUDA graphs as it captures them.  Its continuous-batching scheduler is not
used: that module imports ``zmq``, which is not installed here, and its ``Engine`` serves one
sequence at a time, so the batched step loop of its benchmark is the batched public path there is.

The numbers have the meaning of the other arm's: ``value`` is decoded tokens a second over K steps
timed with CUDA events (host work between steps included, as a step of this engine needs it),
``e2e`` the same loop timed on the host with token ids going in and coming out as Python integers.
"""

from __future__ import annotations

import json
import os
import shutil
import statistics
import sys
import tempfile
import time
from typing import Dict, List

HERE = os.path.dirname(os.path.abspath(__file__))
DEST = os.path.join(HERE, "_ref")


class Unavailable(RuntimeError):
    pass


def _reference_path() -> str:
    """Where to import ``lily`` from.  If the CUDA extension was compiled ahead under another name of
    this same folder (a symlinked checkout), that name is used, so that its build files still match."""
    if not os.path.isfile(os.path.join(DEST, "lily", "engine.py")):
        try:
            sys.path.insert(0, HERE)
            import install_reference
            install_reference.install()
        except Exception as exc:                       # no checkout at hand on this machine
            raise Unavailable(f"the reference is not under baseline/_ref and could not be put there: "
                              f"{type(exc).__name__}: {exc}")
    path = DEST
    stamp = os.path.join(DEST, "_cuda_build", "BUILT_AT")
    if os.path.isfile(stamp):
        built_at = open(stamp).read().strip()
        if built_at and os.path.isdir(built_at) and os.path.realpath(built_at) == os.path.realpath(DEST):
            path = built_at
    return path


def _write_tokenizer(folder: str) -> None:
    tok = {"version": "1.0", "truncation": None, "padding": None, "added_tokens": [], "normalizer": None,
           "pre_tokenizer": {"type": "Whitespace"}, "post_processor": None, "decoder": None,
           "model": {"type": "WordLevel", "vocab": {"<unk>": 0, "a": 1}, "unk_token": "<unk>"}}
    with open(os.path.join(folder, "tokenizer.json"), "w") as f:
        json.dump(tok, f)
    with open(os.path.join(folder, "tokenizer_config.json"), "w") as f:
        json.dump({"tokenizer_class": "PreTrainedTokenizerFast", "unk_token": "<unk>"}, f)


def write_checkpoint(cfg: Dict, folder: str, seed: int = 0, std: float = 0.02) -> int:
    """A model folder in the checkpoint's own tensor names, one shard per layer; returns bytes written."""
    import torch
    from safetensors.torch import save_file

    dev = "cuda" if torch.cuda.is_available() else "cpu"
    gen = torch.Generator(device=dev).manual_seed(seed)
    h, nq, nkv, d = cfg["hidden_size"], cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    inter, vocab, layers = cfg["intermediate_size"], cfg["vocab_size"], cfg["num_hidden_layers"]

    def mat(*shape):
        return (torch.randn(shape, generator=gen, device=dev, dtype=torch.float32) * std).to(torch.bfloat16).cpu()

    def ones(n):
        return torch.ones(n, dtype=torch.bfloat16)

    index, total = {}, 0

    def shard(name, tensors):
        nonlocal total
        save_file(tensors, os.path.join(folder, name))
        for k, v in tensors.items():
            index[k] = name
            total += v.numel() * v.element_size()

    shard("model-embed.safetensors", {"model.embed_tokens.weight": mat(vocab, h), "model.norm.weight": ones(h)})
    for i in range(layers):
        p = f"model.layers.{i}"
        t = {f"{p}.self_attn.q_proj.weight": mat(nq * d, h), f"{p}.self_attn.k_proj.weight": mat(nkv * d, h),
             f"{p}.self_attn.v_proj.weight": mat(nkv * d, h), f"{p}.self_attn.o_proj.weight": mat(h, nq * d),
             f"{p}.mlp.gate_proj.weight": mat(inter, h), f"{p}.mlp.up_proj.weight": mat(inter, h),
             f"{p}.mlp.down_proj.weight": mat(h, inter), f"{p}.input_layernorm.weight": ones(h),
             f"{p}.post_attention_layernorm.weight": ones(h)}
        if "Qwen3" in cfg["architectures"][0]:
            t[f"{p}.self_attn.q_norm.weight"] = ones(d)
            t[f"{p}.self_attn.k_norm.weight"] = ones(d)
        shard(f"model-layer-{i:03d}.safetensors", t)
    if not cfg.get("tie_word_embeddings"):
        shard("model-head.safetensors", {"lm_head.weight": mat(vocab, h)})
    with open(os.path.join(folder, "model.safetensors.index.json"), "w") as f:
        json.dump({"metadata": {"total_size": total}, "weight_map": index}, f)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    _write_tokenizer(folder)
    return total


def _scratch_folder(need_bytes: int) -> str:
    roots = [os.environ.get("LILY_BENCH_TMP"), tempfile.gettempdir(), "/dev/shm"]
    for root in roots:
        if root and os.path.isdir(root) and shutil.disk_usage(root).free > need_bytes * 1.1:
            return tempfile.mkdtemp(prefix="lily_ref_ckpt_", dir=root)
    raise Unavailable(f"no temporary folder with {need_bytes / 1e9:.0f} GB free for the reference's checkpoint")


def run(a, cfg: Dict, context: int, prefill_tokens: int, clock_sampler, rounds: int) -> Dict:
    """Measures the reference; returns the fields of the JSON line that differ from arm to arm."""
    path = _reference_path()
    os.environ.setdefault("HF_HUB_OFFLINE", "1")
    os.environ.setdefault("TRANSFORMERS_OFFLINE", "1")
    build_dir = os.path.join(path, "_cuda_build")
    if os.path.isdir(build_dir):
        os.environ.setdefault("LILY_CUDA_BUILD_DIR", build_dir)
        os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0")
    sys.path.insert(0, path)
    import torch

    if not torch.cuda.is_available():
        raise Unavailable("no CUDA device")
    torch.cuda.set_device(0)
    from lily.engine import Engine, EngineConfig
    from lily.model_executor.forward_batch_info import ForwardBatch

    h, layers = cfg["hidden_size"], cfg["num_hidden_layers"]
    params = layers * (h * (cfg["num_attention_heads"] + 2 * cfg["num_key_value_heads"]) * cfg["head_dim"]
                       + cfg["num_attention_heads"] * cfg["head_dim"] * h + 3 * h * cfg["intermediate_size"])
    params += 2 * cfg["vocab_size"] * h
    folder = _scratch_folder(2 * params)
    t0 = time.time()
    try:
        write_checkpoint(cfg, folder, seed=0)
        print(f"reference arm: checkpoint written in {time.time() - t0:.0f} s", file=sys.stderr, flush=True)
        max_batch = max(a.batch, 8 if a.skip_points else 64)
        t0 = time.time()
        eng = Engine(EngineConfig(folder, dtype="bfloat16", context_length=context, max_running_requests=max_batch,
                                  max_total_tokens=max_batch * (context + 8)))
        load_s = time.time() - t0
    finally:
        shutil.rmtree(folder, ignore_errors=True)
    print(f"reference arm: engine up in {load_s:.0f} s, cuda graphs "
          f"{'on' if eng.runner.cuda_graph_runner is not None else 'off'}", file=sys.stderr, flush=True)
    runner, device, vocab = eng.runner, eng.device, cfg["vocab_size"]
    g = torch.Generator().manual_seed(1)

    def ids(n: int) -> List[int]:
        return torch.randint(0, vocab, (n,), generator=g).tolist()

    def sync():
        torch.cuda.synchronize(device)

    # ---- prefill: one request of `prefill_tokens` tokens ------------------------------------------
    prompt = ids(prefill_tokens)

    @torch.inference_mode()
    def prefill_once():
        idx = eng._new_seq()
        try:
            loc = eng._alloc(idx, 0, prefill_tokens)
            fb = ForwardBatch.for_extend([prompt], [0], [idx], device, out_cache_loc=loc)
            runner.forward(fb)
        finally:
            sync()
            eng._release(idx, prefill_tokens)

    for _ in range(3):
        prefill_once()
    times = []
    for _ in range(5):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        sync()
        e0.record()
        prefill_once()
        e1.record()
        sync()
        times.append(e0.elapsed_time(e1))
    prefill_ms = statistics.fmean(times)

    # ---- decode ----------------------------------------------------------------------------------
    @torch.inference_mode()
    def decode_point(batch: int, k: int, w: int, r: int):
        total = w + 2 * r * k
        start_len = context - total - 1
        idxs = [eng._new_seq() for _ in range(batch)]
        seq = [0] * batch
        try:
            for i in range(batch):
                p = ids(start_len)
                loc = eng._alloc(idxs[i], 0, start_len)
                runner.forward(ForwardBatch.for_extend([p], [0], [idxs[i]], device, out_cache_loc=loc))
                seq[i] = start_len
            state = {"toks": [ids(1)[0] for _ in range(batch)]}

            def one():
                locs = torch.cat([eng._alloc(idxs[i], seq[i], 1) for i in range(batch)])
                fb = ForwardBatch.for_decode(state["toks"], [s + 1 for s in seq], idxs, device, out_cache_loc=locs)
                out = runner.forward(fb)
                for i in range(batch):
                    seq[i] += 1
                state["toks"] = [int(t) for t in torch.argmax(out.next_token_logits, dim=-1)]

            for _ in range(w):
                one()
            dev_ms, host_ms = [], []
            with clock_sampler() as clocks:
                for _ in range(r):
                    clocks.region = "value"
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    sync()
                    e0.record()
                    for _ in range(k):
                        one()
                    e1.record()
                    sync()
                    dev_ms.append(e0.elapsed_time(e1) / k)
                    clocks.region = "e2e"
                    t = time.perf_counter()
                    for _ in range(k):
                        one()
                    sync()
                    host_ms.append((time.perf_counter() - t) * 1e3 / k)
                clocks.region = "idle"
            return statistics.median(dev_ms), statistics.median(host_ms), start_len + w + r * k, clocks.summary()
        finally:
            sync()
            for i in range(batch):
                eng._release(idxs[i], seq[i])

    steps, warmup = max(1, a.steps), max(3, a.warmup)
    ms, host_ms, mean_ctx, clocks = decode_point(a.batch, steps, warmup, rounds)
    points = {}
    if not a.skip_points:
        for b in (1, 64):
            pms, _, _, _ = decode_point(b, min(steps, 32), warmup, 3)      # medians over three rounds, as the other arm
            points[f"decode_b{b}"] = round(b / pms * 1e3, 1)
    graphs = eng.runner.cuda_graph_runner is not None
    return {"ms": ms, "e2e_ms": host_ms, "mean_ctx": mean_ctx, "clocks": clocks, "points": points,
            "prefill_ms": prefill_ms, "load_s": load_s, "cuda_graphs": graphs,
            "h2d_bytes_per_step": 8 * (4 * a.batch), "d2h_bytes_per_step": 8 * a.batch}
