"""CPU-side checks of the C-ABI library: it loads without a GPU, exports every symbol the
header declares, and its host scalar state machine equals the oracle's for any call history.
No kernel is launched here."""
import ctypes as C
import re
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parents[1]


@pytest.fixture(scope="module")
def lib():
    from slideformer_b200 import _lib
    return _lib.load()


def test_header_symbols_are_exported_and_bound(lib):
    from slideformer_b200 import _lib
    header = (ROOT / "include" / "slideformer_b200.h").read_text()
    header = re.sub(r"/\*.*?\*/", "", header, flags=re.S)
    declared = set(re.findall(r"\b(sf_[a-z0-9_]+)\s*\(", header))
    assert declared, "no declarations parsed"
    for name in declared:
        assert hasattr(lib, name), f"{name} is declared in the header but not exported"
    assert declared == set(_lib.SIGNATURES), "ctypes table and header disagree"
    assert lib.sf_abi_version() == _lib.SF_ABI_VERSION


def test_struct_layout_matches_header():
    from slideformer_b200._lib import SfAdamScalars, SfGradStats
    assert C.sizeof(SfAdamScalars) == 56 and SfAdamScalars.grad_scale.offset == 40 and SfAdamScalars.grad_stats.offset == 48
    assert C.sizeof(SfGradStats) == 256 and SfGradStats.nonfinite.offset == 128


def scal(lib, oid, *a):
    from slideformer_b200._lib import SfAdamScalars, check
    s = SfAdamScalars()
    check(lib.sf_adam_scalars(oid, *a, C.byref(s)))
    return s


FIELDS = [("beta1", "betta1"), ("beta2", "betta2"), ("omb1", "omb1"), ("omb2", "omb2"), ("bc2", "bc2"),
          ("eps", "eps"), ("step_size", "step_size"), ("w_decay", "w_decay"), ("weight_decay", "weight_decay"),
          ("adamw_mode", "adamw_mode")]


def same(s, c):
    for a, b in FIELDS:
        x, y = getattr(s, a), getattr(c, b)
        if isinstance(x, float):
            assert np.float32(x).view(np.uint32) == np.float32(y).view(np.uint32), (a, x, y)
        else:
            assert x == y, (a, x, y)


def test_scalar_state_machine_matches_oracle(lib, oracle):
    """Running product on the first call of a step, pow() on repeats, jumps and beta changes
    (cpu_adam.h:57-76)."""
    from slideformer_b200._lib import check
    oid = 9001
    check(lib.sf_adam_create(oid, 1e-5, 0.9, 0.999, 1e-8, 0.01, 1, 0))
    orc = oracle.OracleAdam(1e-5, 0.9, 0.999, 1e-8, 0.01, True)
    rng = np.random.default_rng(0)
    history = []
    step = 0
    for _ in range(400):
        r = rng.random()
        if r < 0.5:
            step += 1                      # normal advance -> product path
        elif r < 0.8:
            pass                           # same step again (another parameter / chunk) -> pow path
        elif r < 0.9:
            step += int(rng.integers(2, 50))  # skipped steps -> pow path
        else:
            step = max(1, step - 1)
        b1, b2 = (0.9, 0.999) if rng.random() < 0.9 else (0.8, 0.95)
        lr = float(rng.choice([1e-5, 3e-4, 0.01]))
        bc = int(rng.random() < 0.8)
        wd = float(rng.choice([0.0, 0.01, 0.1]))
        history.append((step, lr, b1, b2, 1e-8, wd, bc))
    for h in history:
        same(scal(lib, oid, *h), orc.scalars(*h))
    check(lib.sf_adam_destroy(oid))


def test_long_run_product_path(lib, oracle):
    from slideformer_b200._lib import check
    oid = 9002
    check(lib.sf_adam_create(oid, 1e-3, 0.9, 0.999, 1e-8, 0.0, 1, 0))
    orc = oracle.OracleAdam(1e-3, 0.9, 0.999, 1e-8, 0.0, True)
    for step in range(1, 3000):
        h = (step, 1e-3, 0.9, 0.999, 1e-8, 0.0, 1)
        same(scal(lib, oid, *h), orc.scalars(*h))
    check(lib.sf_adam_destroy(oid))


def test_error_codes_without_gpu(lib):
    from slideformer_b200 import _lib
    s = _lib.SfAdamScalars()
    assert lib.sf_adam_scalars(123456, 1, 1e-3, 0.9, 0.999, 1e-8, 0.0, 1, C.byref(s)) == _lib.SF_ERR_UNKNOWN_ID
    assert b"123456" in lib.sf_last_error()
    assert lib.sf_adam_scalars(0, 1, 1e-3, 0.9, 0.999, 1e-8, 0.0, 1, None) == _lib.SF_ERR_NULL
    assert lib.sf_adam_create(77, 1e-3, 0.9, 0.999, 1e-8, 0.0, 1, 0) == 0
    # bad dtype code and NULL buffers are rejected before any CUDA call and before the state moves
    assert lib.sf_adam_update(77, 1, 1e-3, 0.9, 0.999, 1e-8, 0.0, 1, None, None, 5, None, None, None, 0, None) == _lib.SF_ERR_DTYPE
    assert lib.sf_adam_update(77, 1, 1e-3, 0.9, 0.999, 1e-8, 0.0, 1, None, None, 0, None, None, None, 16, None) == _lib.SF_ERR_NULL
    # n == 0 is a valid call (the reference accepts empty chunks) and needs no device
    assert lib.sf_adam_update(77, 1, 1e-3, 0.9, 0.999, 1e-8, 0.0, 1, None, None, 0, None, None, None, 0, None) == 0
    assert lib.sf_adam_step_sharded(C.byref(s), None, None, 0, 0, None, None, None, 0, 0, None) == _lib.SF_ERR_ARG
    assert lib.sf_adam_step_sharded(C.byref(s), None, None, 17, 0, None, None, None, 0, 0, None) == _lib.SF_ERR_ARG
    assert lib.sf_adam_step_sharded_push(C.byref(s), None, None, None, 0, 0, None, None, 0, 0, None) == _lib.SF_ERR_ARG
    assert lib.sf_adam_step_sharded_push(C.byref(s), None, None, None, 2, 9, None, None, 0, 0, None) == _lib.SF_ERR_DTYPE
    assert lib.sf_adam_step_sharded_push(C.byref(s), None, None, None, 2, 0, None, None, 16, 16, None) == _lib.SF_ERR_NULL
    assert lib.sf_dp_mean(None, 2, 0, None, 16, None) == _lib.SF_ERR_NULL
    assert lib.sf_dp_mean(None, 2, 0, None, 0, None) == 0
    assert lib.sf_adam_update_dp_static(77, 1, 1e-3, 0.9, 0.999, 1e-8, 0.0, 1, None, None, 2, 0, None, None, None,
                                        _lib.SF_STATIC_SCRATCH_MAX_ELEMS + 1, None) == _lib.SF_ERR_SIZE
    assert lib.sf_adam_update_host(77, 1, 1e-3, 0.9, 0.999, 1e-8, 0.0, 1, None, None, 0, 0, None, None, None,
                                   0, 24, 0, None, 0, None) == _lib.SF_ERR_ARG  # chunk not a multiple of 16
    assert lib.sf_adam_host_scratch_bytes(1024, 0, 1) == 2 * (3 * 4096 + 2048)
    assert lib.sf_adam_host_scratch_bytes(1024, 0, 0) == 2 * (3 * 4096)
    assert lib.sf_set_tuning(7, -1) == _lib.SF_ERR_ARG
    assert lib.sf_adam_destroy(77) == 0
    assert lib.sf_adam_destroy(77) == 0  # unknown ids are ignored


def test_layer_adam_host_rules_without_gpu():
    """Pageable host parameters are refused: the package has no CPU arithmetic."""
    import torch
    from slideformer_b200 import LayerAdam
    opt = LayerAdam(lr=1e-3)
    assert opt.add_layer_params(0, []) == -1
    with pytest.raises(RuntimeError, match="pinned"):
        opt.add_layer_params(0, [torch.nn.Parameter(torch.zeros(8))])
    with pytest.raises(RuntimeError, match="float32"):
        opt.add_layer_params(0, [torch.nn.Parameter(torch.zeros(8, dtype=torch.bfloat16))])
    with pytest.raises(NotImplementedError):
        LayerAdam(nvme_offload_fraction=0.5)
    opt.update_learning_rate(5e-4)
    assert opt.defaults["lr"] == 5e-4
    assert set(opt.defaults) == {"lr", "bias_correction", "betas", "eps", "weight_decay", "adamw_mode"}
    # step_chunk with a plain dict and pageable CPU tensors: refused, never computed on the CPU
    z = torch.zeros(4)
    with pytest.raises(RuntimeError, match="pinned"):
        opt.step_chunk(z, z.clone(), z.clone(), z.clone(), dict(opt.defaults, step=1))


C_CLIENT = r"""
#include <stdio.h>
#include <string.h>
#include "slideformer_b200.h"
int main(void) {
    SfAdamScalars s;
    if (sf_abi_version() != SF_ABI_VERSION) return 2;
    if (sf_adam_create(5, 1e-5f, 0.9f, 0.999f, 1e-8f, 0.01f, 1, 0) != SF_OK) return 3;
    if (sf_adam_scalars(5, 1, 1e-5f, 0.9f, 0.999f, 1e-8f, 0.01f, 1, &s) != SF_OK) return 4;
    if (sf_adam_scalars(6, 1, 1e-5f, 0.9f, 0.999f, 1e-8f, 0.01f, 1, &s) != SF_ERR_UNKNOWN_ID) return 5;
    if (strstr(sf_last_error(), "6") == NULL) return 6;
    if (sf_adam_update(5, 2, 1e-5f, 0.9f, 0.999f, 1e-8f, 0.01f, 1, NULL, NULL, SF_GRAD_BF16, NULL, NULL, NULL, 0, NULL) != SF_OK) return 7;
    printf("%.9g %.9g %.9g %d %u\n", s.omb1, s.bc2, s.step_size, s.adamw_mode, (unsigned)SF_STATIC_SCRATCH_MAX_ELEMS);
    return sf_adam_destroy(5);
}
"""


def test_header_is_plain_c_and_links_from_c(tmp_path, oracle):
    """The boundary is a C ABI: a C99 translation unit includes the header and links the library."""
    import subprocess
    from slideformer_b200 import _lib
    _lib.load()
    src = tmp_path / "client.c"
    src.write_text(C_CLIENT)
    exe = tmp_path / "client"
    lib_dir = _lib.LIB_PATH.parent
    subprocess.check_call(["/usr/bin/gcc", "-std=c99", "-Wall", "-Werror", "-pedantic", f"-I{ROOT / 'include'}", str(src),
                           "-o", str(exe), f"-L{lib_dir}", "-lslideformer_b200", f"-Wl,-rpath,{lib_dir}"])
    out = subprocess.run([str(exe)], capture_output=True, text=True)
    assert out.returncode == 0, (out.returncode, out.stdout, out.stderr)
    omb1, bc2, step_size, adamw, max_elems = out.stdout.split()
    c = oracle.OracleAdam(1e-5, 0.9, 0.999, 1e-8, 0.01, True).scalars(1, 1e-5, 0.9, 0.999, 1e-8, 0.01, True)
    assert np.float32(float(omb1)) == np.float32(c.omb1) and np.float32(float(bc2)) == np.float32(c.bc2)
    assert np.float32(float(step_size)) == np.float32(c.step_size) and adamw == "1" and int(max_elems) == 4 << 20
