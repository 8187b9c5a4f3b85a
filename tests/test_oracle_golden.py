"""The C restatement against the golden vectors produced by the compiled reference kernel.

Bit-exact on p, m, v for every case; the bf16 copy is bit-exact too (no NaN in these cases).
"""
import numpy as np
import pytest

from golden_cases import REFT, REFTEST_CHUNK, REFTEST_SIZES, TRAJ_CASES, reftest_lr


def bits(a):
    return a.view(np.uint32) if a.dtype == np.float32 else a


@pytest.mark.parametrize("name", sorted(TRAJ_CASES))
def test_trajectory_matches_reference_bits(name, golden, oracle):
    hp, adamw, bc, steps = TRAJ_CASES[name]
    p = golden[f"{name}/p0"].copy()
    n = p.size
    m = np.zeros(n, np.float32)
    v = np.zeros(n, np.float32)
    out = np.zeros(n, np.uint16)
    g_all = golden[f"{name}/g"]
    bounds = golden[f"{name}/bounds"]
    opt = oracle.OracleAdam(hp["lr"], hp["b1"], hp["b2"], hp["eps"], hp["wd"], adamw)
    for step in range(1, steps + 1):
        g = g_all[step - 1]
        for a, b in zip(bounds[:-1], bounds[1:]):
            if b > a:
                opt.adam_update(step, hp["lr"], hp["b1"], hp["b2"], hp["eps"], hp["wd"], bc,
                                p[a:b], g[a:b], m[a:b], v[a:b], out[a:b])
        tag = f"{name}/s{step}"
        if f"{tag}/p" in golden:
            assert np.array_equal(bits(p), bits(golden[f"{tag}/p"]))
            assert np.array_equal(bits(m), bits(golden[f"{tag}/m"]))
            assert np.array_equal(bits(v), bits(golden[f"{tag}/v"]))
            assert np.array_equal(out, golden[f"{tag}/bf16"])


@pytest.mark.parametrize("dt", ["f32", "bf16"])
def test_reference_dp_test_sequence(dt, golden, oracle):
    """Call sequence of the reference's own test (19/3/0 elements, chunks of 5, shared optimizer)."""
    opt = oracle.OracleAdam(0.01, REFT["b1"], REFT["b2"], REFT["eps"], REFT["wd"], True)
    ps = [golden[f"reftest/{dt}/L{i}/p0"].copy() for i in range(3)]
    ms = [np.zeros_like(p) for p in ps]
    vs = [np.zeros_like(p) for p in ps]
    for step in range(1, 6):
        lr = reftest_lr(step)
        for li, size in enumerate(REFTEST_SIZES):
            rows = golden[f"reftest/{dt}/L{li}/g{step}"]
            for s in range(0, size, REFTEST_CHUNK):
                e = min(s + REFTEST_CHUNK, size)
                mean = oracle.rank_mean(np.ascontiguousarray(rows[:, s:e]))
                opt.adam_update(step, lr, REFT["b1"], REFT["b2"], REFT["eps"], REFT["wd"], True,
                                ps[li][s:e], mean, ms[li][s:e], vs[li][s:e])
    for li in range(3):
        assert np.array_equal(bits(ps[li]), bits(golden[f"reftest/{dt}/L{li}/p"]))
        assert np.array_equal(bits(ms[li]), bits(golden[f"reftest/{dt}/L{li}/m"]))
        assert np.array_equal(bits(vs[li]), bits(golden[f"reftest/{dt}/L{li}/v"]))


def test_reference_dp_test_tolerance_vs_torch_adamw(golden):
    """The reference pins this path to torch.optim.AdamW at rtol 1e-6 / atol 1e-7
    (multi_gpu/tests/test_shared_data_parallel.py:89); the golden vectors meet that."""
    import torch
    for li, size in enumerate(REFTEST_SIZES):
        ref = torch.nn.Parameter(torch.from_numpy(golden[f"reftest/f32/L{li}/p0"].copy()))
        opt = torch.optim.AdamW([ref], lr=0.01, betas=(0.8, 0.95), eps=1e-6, weight_decay=0.1, foreach=False)
        for step in range(1, 6):
            rows = torch.from_numpy(golden[f"reftest/f32/L{li}/g{step}"].copy())
            opt.param_groups[0]["lr"] = reftest_lr(step)
            ref.grad = rows.float().mean(0) if size else torch.zeros(0)
            opt.step()
        torch.testing.assert_close(torch.from_numpy(golden[f"reftest/f32/L{li}/p"].copy()), ref.data,
                                   rtol=1e-6, atol=1e-7)


def test_bf16_cast_rne_and_nan(oracle):
    import torch
    gen = torch.Generator().manual_seed(7)
    x = torch.randn(100003, generator=gen) * 3
    x[:6] = torch.tensor([float("inf"), -float("inf"), 0.0, -0.0, 1e-40, -3e-39])
    got = oracle.f32_to_bf16(x.numpy())
    want = x.to(torch.bfloat16).view(torch.uint16).numpy()
    assert np.array_equal(got, want)
    # ties: exactly halfway mantissas round to even
    u = np.array([0x3F808000, 0x3F818000, 0x3F80FFFF, 0x7F7FFFFF], dtype=np.uint32)
    assert oracle.f32_to_bf16(u.view(np.float32)).tolist() == [0x3F80, 0x3F82, 0x3F81, 0x7F80]
    # every NaN becomes the canonical quiet NaN 0x7FC0 (simd.h:74-83; c10::BFloat16 scalar cast)
    nan = np.array([0x7FC00000, 0xFFC00000, 0x7F800001, 0x7FFFFFFF], dtype=np.uint32).view(np.float32)
    assert oracle.f32_to_bf16(nan).tolist() == [0x7FC0] * 4


def test_rank_mean_order(oracle):
    rows = np.array([[1e8], [1.0], [-1e8]], dtype=np.float32)
    # (0 + 1e8 + 1) - 1e8 in fp32 loses the 1: order matters and must be rank order
    assert oracle.rank_mean(rows)[0] == np.float32(0.0)
    rows2 = np.array([[1e8], [-1e8], [1.0]], dtype=np.float32)
    assert oracle.rank_mean(rows2)[0] == np.float32(1.0) / np.float32(3.0)
