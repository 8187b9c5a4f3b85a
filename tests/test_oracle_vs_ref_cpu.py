"""The C restatement (oracle/) against the reference's own compiled kernel (oracle/_ref/), directly.

oracle/_ref/cpu_adam.so is built from the reference's two source files by oracle/build_ref.py
wherever the reference checkout is present; it travels with the tree but is not committed, so
these tests skip where it is absent (or where the host lacks AVX-512).  They pin the oracle at
sizes the committed golden vectors do not reach: 2^20 + 13 elements over several steps and
hyper-parameter sets, and the full 218,112,000-element layer of the benchmark configuration.
"""
import numpy as np
import pytest
import torch


@pytest.fixture(scope="module")
def ref():
    from oracle import build_ref
    mod = build_ref.load()
    if mod is None:
        pytest.skip("oracle/_ref/cpu_adam.so is absent or this host lacks AVX-512")
    return mod


def _bits(a):
    return a.view(np.uint32)


def _run(ref, oracle, n, steps, hp, adamw, bc, gdtype, oid, calls_per_step=1):
    lr, b1, b2, eps, wd = hp
    gen = torch.Generator().manual_seed(n % 1000 + oid)
    p = torch.empty(n).normal_(0, 0.02, generator=gen)
    if n > 8192:
        p[-8192:] = 1.0
    m, v = torch.zeros(n), torch.zeros(n)
    po, mo, vo = p.numpy().copy(), np.zeros(n, np.float32), np.zeros(n, np.float32)
    ref.create_adam(oid, lr, b1, b2, eps, wd, adamw, False)
    orc = oracle.OracleAdam(lr, b1, b2, eps, wd, adamw)
    cuts = np.linspace(0, n, calls_per_step + 1).astype(np.int64)
    try:
        for step in range(1, steps + 1):
            g = torch.empty(n).normal_(0, 1e-3, generator=gen).to(gdtype)
            gnp = g.view(torch.int16).numpy().view(np.uint16) if gdtype == torch.bfloat16 else g.numpy()
            if gdtype == torch.float16 and step == 1:
                # exercise subnormal, signed-zero and infinite halves as well
                gnp[:8] = np.array([0.0, -0.0, 6e-8, -6e-5, 65504.0, np.inf, 1e-7, -1.0], dtype=np.float16)
            for a, b in zip(cuts[:-1], cuts[1:]):
                ref.adam_update(oid, step, lr, b1, b2, eps, wd, bc, p[a:b], g[a:b], m[a:b], v[a:b])
                orc.adam_update(step, lr, b1, b2, eps, wd, bc, po[a:b], gnp[a:b], mo[a:b], vo[a:b])
            for name, x, y in (("p", p, po), ("m", m, mo), ("v", v, vo)):
                bad = np.nonzero(_bits(x.numpy()) != _bits(y))[0]
                assert bad.size == 0, f"step {step} {name}: {bad.size} of {n} differ, first at {bad[0]}"
    finally:
        ref.destroy_adam(oid)


@pytest.mark.parametrize("gdtype", [torch.bfloat16, torch.float32, torch.float16])
@pytest.mark.parametrize("hp,adamw,bc", [((1e-5, 0.9, 0.999, 1e-8, 0.01), True, True),
                                         ((0.01, 0.8, 0.95, 1e-6, 0.1), False, True),
                                         ((1e-3, 0.9, 0.999, 1e-8, 0.0), True, False)])
def test_oracle_equals_compiled_reference_1m(ref, oracle, hp, adamw, bc, gdtype):
    """n = 2^20 + 13: vector body, a 13-element scalar tail, 5 steps, three calls per step (so
    the pow() branch of the scalar state machine runs too)."""
    _run(ref, oracle, (1 << 20) + 13, 5, hp, adamw, bc, gdtype, oid=5100, calls_per_step=3)


def test_oracle_equals_compiled_reference_full_layer(ref, oracle):
    """The benchmark's layer, every element, two steps."""
    _run(ref, oracle, 218_112_000, 2, (1e-5, 0.9, 0.999, 1e-8, 0.01), True, True, torch.bfloat16, oid=5101)
