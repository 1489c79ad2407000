"""The router's exp() must return the host C library's expf bits (csrc/expf_compat.h).  The header
compiles as plain C; this test builds it with gcc and compares it with libm over a dense sample of the
router's input range (x = logit - max <= 0) and around every threshold."""
import ctypes as C
import subprocess
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent.parent
SHIM = r'''
#include "expf_compat.h"
static uint64_t tab[UOCR_EXPF_N]; static int ready;
void shim_expf(const float *x, float *y, long n) {
    if (!ready) { uocr_expf_table_init(tab); ready = 1; }
    for (long i = 0; i < n; ++i) y[i] = uocr_expf_compat(x[i], tab);
}
void libm_expf(const float *x, float *y, long n) { for (long i = 0; i < n; ++i) y[i] = expf(x[i]); }
'''


def test_expf_bits_equal_libm(tmp_path):
    src = tmp_path / "shim.c"
    src.write_text(SHIM)
    lib_path = tmp_path / "shim.so"
    subprocess.run(["gcc", "-O2", "-shared", "-fPIC", f"-I{ROOT / 'unlimitedocr.c_b200' / 'csrc'}", "-o", str(lib_path),
                    str(src), "-lm"], check=True)
    lib = C.CDLL(str(lib_path))
    fp = np.ctypeslib.ndpointer(np.float32, flags="C_CONTIGUOUS")
    for fn in (lib.shim_expf, lib.libm_expf):
        fn.argtypes = [fp, fp, C.c_long]
    rng = np.random.default_rng(0)
    edge = np.array([0.0, -0.0, -1e-30, -88.0, -87.3365, -87.4, -103.9, -103.972, -103.98, -104.0, -1e9, -np.inf,
                     0.5, 1.0, 88.7, 88.8, np.inf], np.float32)
    around = np.concatenate([np.nextafter(edge, np.float32(-np.inf)), np.nextafter(edge, np.float32(np.inf))])
    # every 64th negative float from -0 down to -128, plus random draws shaped like logit differences
    grid = np.arange(0x80000000, 0xC3000000, 64, dtype=np.uint64).astype(np.uint32).view(np.float32)
    rand = -np.abs(rng.standard_normal(4_000_000).astype(np.float32) * rng.choice([0.1, 1, 8, 40], 4_000_000).astype(np.float32))
    x = np.ascontiguousarray(np.concatenate([edge, around, grid, rand]), np.float32)
    a, b = np.empty_like(x), np.empty_like(x)
    lib.shim_expf(x, a, x.size)
    lib.libm_expf(x, b, x.size)
    mism = np.flatnonzero(a.view(np.uint32) != b.view(np.uint32))
    # A host whose libm was built without fused multiply-add may differ by one ulp on isolated inputs
    # (two in the whole float range); anything more is a real disagreement.
    assert mism.size <= 2, (mism.size, x[mism[:5]], a[mism[:5]], b[mism[:5]])
    assert np.all(np.abs(a[mism].view(np.int32).astype(np.int64) - b[mism].view(np.int32)) <= 1)
