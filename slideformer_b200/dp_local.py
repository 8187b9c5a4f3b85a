"""The data-parallel kernels on one GPU, with `world` local buffers standing in for the peers.

    python -m slideformer_b200.dp_local --world 8 --n 16000000 --steps 5 [--entry push|pull] [--vec 8]

sf_adam_step_sharded_push / sf_adam_step_sharded take arrays of device pointers and do not care
whether a pointer is local or peer-mapped, so the very kernels the multi-GPU runs launch can be
run, timed and profiled on a single GPU.  There the gradient pulls and the bf16 pushes are HBM
traffic: per parameter 26 bytes of fp32 state, 2 * world bytes of gradients read and (push)
2 * world bytes of bf16 weights written.  Prints one JSON line.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import sys

import torch

from . import _lib


def run(world: int, n: int, steps: int, entry: str = "push", vec: int = 8, warmup: int = 3, device="cuda:0") -> dict:
    lib = _lib.load()
    dev = torch.device(device)
    torch.cuda.set_device(dev)
    _lib.check(lib.sf_set_push_tuning(vec, 1))
    gen = torch.Generator(device=dev).manual_seed(0)
    p = torch.empty(n, device=dev).normal_(0, 0.02, generator=gen)
    m, v = torch.zeros(n, device=dev), torch.zeros(n, device=dev)
    grads = [torch.empty(n, device=dev).normal_(0, 1e-3, generator=gen).to(torch.bfloat16) for _ in range(world)]
    outs = [torch.empty(n, device=dev, dtype=torch.bfloat16) for _ in range(world if entry == "push" else 1)]
    peers = (C.c_void_p * world)(*[g.data_ptr() for g in grads])
    optrs = (C.c_void_p * len(outs))(*[o.data_ptr() for o in outs])
    oid = 991000 + world
    hp = (1e-5, 0.9, 0.999, 1e-8, 0.01)
    _lib.check(lib.sf_adam_create(oid, *hp, 1, 0))
    stream = torch.cuda.current_stream().cuda_stream
    sc = _lib.SfAdamScalars()

    def one(step):
        _lib.check(lib.sf_adam_scalars(oid, step, *hp, 1, C.byref(sc)))
        if entry == "push":
            _lib.check(lib.sf_adam_step_sharded_push(C.byref(sc), p.data_ptr(), peers, optrs, world, _lib.SF_GRAD_BF16,
                                                     m.data_ptr(), v.data_ptr(), n, n & ~15, stream))
        else:
            _lib.check(lib.sf_adam_step_sharded(C.byref(sc), p.data_ptr(), peers, world, _lib.SF_GRAD_BF16, m.data_ptr(),
                                                v.data_ptr(), outs[0].data_ptr(), n, n & ~15, stream))
    try:
        for s in range(1, warmup + 1):
            one(s)
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for s in range(warmup + 1, warmup + steps + 1):
            one(s)
        b.record()
        torch.cuda.synchronize()
    finally:
        lib.sf_adam_destroy(oid)
        lib.sf_set_push_tuning(8, 1)
    ms = a.elapsed_time(b) / steps
    bytes_per_param = 26 + 2 * world + 2 * len(outs)
    return {"entry": "sf_adam_step_sharded_push" if entry == "push" else "sf_adam_step_sharded", "world": world, "n": n,
            "vec": vec, "steps": steps, "ms": ms, "bytes_per_param_local": bytes_per_param,
            "hbm_gbs": bytes_per_param * n / (ms * 1e-3) / 1e9, "peers": "local buffers of one GPU"}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--world", type=int, default=8)
    ap.add_argument("--n", type=int, default=16_000_000)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--entry", default="push", choices=["push", "pull"])
    ap.add_argument("--vec", type=int, default=8, choices=[4, 8])
    a = ap.parse_args(argv)
    print(json.dumps(run(a.world, a.n, a.steps, a.entry, a.vec, a.warmup)))
    return 0


if __name__ == "__main__":
    sys.exit(main())
