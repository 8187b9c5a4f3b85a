"""Generate tests/golden/layer_adam_golden.npz from the COMPILED REFERENCE kernel.

Run where the reference checkout is mounted (it cannot travel to the GPU machine):

    python oracle/build_ref.py            # builds oracle/_ref/cpu_adam.so from the reference sources
    python tests/golden/make_golden.py    # writes the .npz next to this file
    python tests/golden/make_golden.py --check-march   # also proves -march does not change results

Every output array in the fixture was produced by the reference's `adam_update`
(optimizer/layer_adam/csrc/cpu_adam.cpp:8-13) on torch CPU tensors, and every bf16 copy by
torch's CPU float32 -> bfloat16 `copy_` (transformer_layer.py:296-305).  The C restatement
and the CUDA path are both tested against these arrays.

Cases
  cfg0/<n>      hyper-parameters of the single-layer benchmark config (lr 1e-5, betas (0.9, 0.999),
                eps 1e-8, wd 0.01, AdamW, bias correction); p ~ N(0, 0.02), bf16 g ~ N(0, 1e-3),
                10 steps, one call per step.  n in 0, 1, 15, 16, 17, 1000, 4099.
  chunk/<n>     same hyper-parameters, each step split into two calls (the second call of a
                step takes the pow() branch of the scalar state machine).  n = 16411, 3 steps.
  modes/<name>  L2 mode, no bias correction, zero weight decay, fp32 gradients.  n = 1007, 4 steps.
  reftest/<dt>  the exact call sequence of multi_gpu/tests/test_shared_data_parallel.py:27-93 with
                --native for world size 2: layers of 19, 3 and 0 elements, chunks of 5, one shared
                optimizer id, five steps, lr 0.01 -> 0.003 at step 3, betas (0.8, 0.95), eps 1e-6,
                wd 0.1, gradients sin(0.13 i + peer + 0.2 step) * 0.1 averaged in fp32 in rank order.
"""
from __future__ import annotations

import argparse
import sys
import tempfile
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
ROOT = HERE.parents[1]
sys.path.insert(0, str(ROOT))
from oracle import build_ref  # noqa: E402

CFG0 = dict(lr=1e-5, b1=0.9, b2=0.999, eps=1e-8, wd=0.01)
REFT = dict(b1=0.8, b2=0.95, eps=1e-6, wd=0.1)


def bits16(t: torch.Tensor) -> np.ndarray:
    return t.view(torch.uint16).numpy().copy()


def gen_cfg0_like(ref, n, steps, hp, seed, calls_per_step=1, adamw=True, bc=True,
                  gdtype=torch.bfloat16, snapshot_steps=(1,)):
    gen = torch.Generator().manual_seed(seed)
    p = torch.randn(n, generator=gen) * 0.02
    if n >= 64:
        p[-8:] = 1.0  # norm weights sit at the end of the flat layer
    m = torch.zeros(n)
    v = torch.zeros(n)
    out = {"p0": p.numpy().copy()}
    ref.create_adam(0, hp["lr"], hp["b1"], hp["b2"], hp["eps"], hp["wd"], adamw, False)
    gs = []
    bounds = np.linspace(0, n, calls_per_step + 1).astype(np.int64)
    for step in range(1, steps + 1):
        g = (torch.randn(n, generator=gen) * 1e-3).to(gdtype)
        gs.append(bits16(g) if gdtype == torch.bfloat16 else g.numpy().copy())
        for a, b in zip(bounds[:-1], bounds[1:]):
            if b > a:
                ref.adam_update(0, step, hp["lr"], hp["b1"], hp["b2"], hp["eps"], hp["wd"], bc,
                                p[a:b], g[a:b], m[a:b], v[a:b])
        if step in snapshot_steps or step == steps:
            tag = f"s{step}"
            out[f"{tag}/p"] = p.numpy().copy()
            out[f"{tag}/m"] = m.numpy().copy()
            out[f"{tag}/v"] = v.numpy().copy()
            out[f"{tag}/bf16"] = bits16(p.to(torch.bfloat16))
    ref.destroy_adam(0)
    out["g"] = np.stack(gs) if gs else np.zeros((0, n), np.uint16)
    out["bounds"] = bounds
    return out


def gen_reftest(ref, dtype, world=2):
    sizes = (19, 3, 0)
    chunk = 5
    ref.create_adam(0, 0.01, REFT["b1"], REFT["b2"], REFT["eps"], REFT["wd"], True, False)
    params = [torch.linspace(-0.5, 0.5, s) for s in sizes]
    ms = [torch.zeros(s) for s in sizes]
    vs = [torch.zeros(s) for s in sizes]
    out = {}
    for li, s in enumerate(sizes):
        out[f"L{li}/p0"] = params[li].numpy().copy()
    for step in range(1, 6):
        lr = 0.01 if step < 3 else 0.003
        for li, size in enumerate(sizes):
            grads = [((torch.arange(size) * 0.13 + peer + step * 0.2).sin() * 0.1).to(dtype)
                     for peer in range(world)]
            rows = torch.stack(grads) if size else torch.zeros(world, 0, dtype=dtype)
            out[f"L{li}/g{step}"] = bits16(rows) if dtype == torch.bfloat16 else rows.numpy().copy()
            for start in range(0, size, chunk):
                end = min(start + chunk, size)
                mean = torch.zeros(end - start, dtype=torch.float32)
                for peer in range(world):
                    mean.add_(grads[peer][start:end])
                mean.div_(world)
                ref.adam_update(0, step, lr, REFT["b1"], REFT["b2"], REFT["eps"], REFT["wd"], True,
                                params[li][start:end], mean, ms[li][start:end], vs[li][start:end])
    ref.destroy_adam(0)
    for li in range(len(sizes)):
        out[f"L{li}/p"] = params[li].numpy().copy()
        out[f"L{li}/m"] = ms[li].numpy().copy()
        out[f"L{li}/v"] = vs[li].numpy().copy()
    return out


def generate(ref) -> dict[str, np.ndarray]:
    torch.set_num_threads(1)
    fx: dict[str, np.ndarray] = {}

    def put(prefix, d):
        for k, a in d.items():
            fx[f"{prefix}/{k}"] = a

    for i, n in enumerate((0, 1, 15, 16, 17, 1000, 4099)):
        put(f"cfg0/{n}", gen_cfg0_like(ref, n, 10, CFG0, seed=1000 + i))
    put("chunk/16411", gen_cfg0_like(ref, 16411, 3, CFG0, seed=2000, calls_per_step=2))
    hp_big = dict(lr=1e-3, b1=0.9, b2=0.999, eps=1e-8, wd=0.05)
    put("modes/l2", gen_cfg0_like(ref, 1007, 4, hp_big, seed=3001, adamw=False))
    put("modes/nobc", gen_cfg0_like(ref, 1007, 4, hp_big, seed=3002, bc=False))
    put("modes/nowd", gen_cfg0_like(ref, 1007, 4, dict(hp_big, wd=0.0), seed=3003))
    put("modes/f32g", gen_cfg0_like(ref, 1007, 4, hp_big, seed=3004, gdtype=torch.float32))
    put("reftest/f32", gen_reftest(ref, torch.float32))
    put("reftest/bf16", gen_reftest(ref, torch.bfloat16))
    return fx


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--check-march", action="store_true",
                    help="rebuild the reference with -march=native in a temp dir and require identical fixtures")
    a = ap.parse_args()
    if build_ref.build() is None:
        sys.exit("reference sources not available; cannot generate golden vectors")
    ref = build_ref.load()
    fx = generate(ref)
    if a.check_march:
        import importlib.util
        with tempfile.TemporaryDirectory() as td:
            so = build_ref.build(out_dir=Path(td), march="native", force=True)
            spec = importlib.util.spec_from_file_location("cpu_adam", so)
            mod = importlib.util.module_from_spec(spec)
            spec.loader.exec_module(mod)
            fx2 = generate(mod)
        bad = [k for k in fx if fx[k].tobytes() != fx2[k].tobytes()]
        if bad:
            sys.exit(f"-march changes results for {bad[:5]}")
        print("march check: x86-64-v4 and native builds give identical bits")
    out = HERE / "layer_adam_golden.npz"
    np.savez_compressed(out, **fx)
    print(f"wrote {out} ({out.stat().st_size / 1024:.0f} KiB, {len(fx)} arrays)")


if __name__ == "__main__":
    main()
