"""The C-ABI library loads and exports every symbol include/powerinfer_b200.h declares (no GPU needed)."""
import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "powerinfer_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(pi_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from powerinfer_b200 import build
    path = build.build()
    lib = ctypes.CDLL(path)
    names = declared_symbols()
    assert len(names) >= 15
    for n in names:
        assert hasattr(lib, n), f"{n} declared in the header but not exported"


def test_binding_covers_header_and_host_helpers_work():
    from powerinfer_b200 import _lib, engine, model_file
    assert set(_lib.EXPORTS) | set(engine.ENGINE_EXPORTS) | set(model_file.MODEL_FILE_EXPORTS) == set(declared_symbols())
    assert _lib.lib.pi_version() >= 1
    assert _lib.lib.pi_row_bytes(_lib.PI_TYPE_F16, 4096) == 8192
    assert _lib.lib.pi_row_bytes(_lib.PI_TYPE_Q4_0, 4096) == 2304
    assert _lib.lib.pi_workspace_bytes(4096, 11008, 1) > 0
    # argument validation happens before any CUDA call, so it can be exercised without a device
    rc = _lib.lib.pi_mul_mat(_lib.PI_TYPE_Q4_0, 16, 8, 100, 16, 1, None, 16, 256, 1 << 20, None)
    assert rc == 1 and b"256" in _lib.lib.pi_last_error()


def test_rope_table_matches_reference_recurrence():
    import numpy as np
    from oracle import pio
    from powerinfer_b200 import _lib
    hd, n_pos = 128, 40
    cs = np.empty((n_pos, hd // 2, 2), np.float32)
    _lib.lib.pi_rope_table_host(cs.ctypes.data, n_pos, hd, 10000.0)
    o = pio.Oracle()
    x = np.zeros((1, hd), np.float32)
    x[0, 0::2] = 1.0                      # (1, 0) pairs: rotation gives (cos, sin)
    for pos in (0, 1, 17, 39):
        y = o.rope(x, hd, 1, pos, 10000.0, False)
        assert np.array_equal(y[0, 0::2], cs[pos, :, 0]) and np.array_equal(y[0, 1::2], cs[pos, :, 1])


C_CONSUMER = r"""
#include <stdio.h>
#include <string.h>
#include "powerinfer_b200.h"
int main(void) {
    float cs[4 * 8 * 2];
    if (pi_version() < 1) return 2;
    if (pi_row_bytes(PI_TYPE_Q4_0, 4096) != 2304 || pi_row_bytes(PI_TYPE_F16, 4096) != 8192) return 3;
    if (pi_workspace_bytes(4096, 11008, 4) == 0) return 4;
    pi_rope_table_host(cs, 4, 16, 10000.0f);
    if (cs[0] != 1.0f || cs[1] != 0.0f) return 5;                      /* position 0: cos 1, sin 0 */
    /* argument validation comes before any CUDA call: no device needed */
    if (pi_mul_mat(PI_TYPE_Q4_0, (const void *)16, 8, 100, (const float *)16, 1, NULL, (float *)16, (void *)256, 1u << 20, NULL) != PI_ERR_INVALID) return 6;
    if (strlen(pi_last_error()) == 0) return 7;
    {
        pi_model_file * f = NULL;
        if (pi_model_file_open("/nonexistent/model.gguf", &f) != PI_ERR_INVALID || f != NULL) return 8;
        pi_model_file_close(NULL);
        if (pi_model_file_n_tensors(NULL) != 0) return 9;
    }
    puts("c consumer ok");
    return 0;
}
"""


def test_plain_c99_consumer_compiles_links_and_runs(tmp_path):
    """The header is C (not only C++): a C99 translation unit with -pedantic -Werror includes it, links the library and
    calls the entry points that need no device."""
    import shutil
    import subprocess
    import pytest
    from powerinfer_b200 import build
    if shutil.which("gcc") is None:
        pytest.skip("no gcc")
    lib = build.build()
    src = tmp_path / "consumer.c"
    src.write_text(C_CONSUMER)
    exe = tmp_path / "consumer"
    libdir = os.path.dirname(lib)
    r = subprocess.run(["gcc", "-std=c99", "-pedantic", "-Wall", "-Werror", "-I", os.path.join(ROOT, "include"), str(src), "-o", str(exe),
                        "-L", libdir, "-lpowerinfer_b200", f"-Wl,-rpath,{libdir}"], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-3000:]
    r = subprocess.run([str(exe)], capture_output=True, text=True)
    assert r.returncode == 0 and "c consumer ok" in r.stdout, (r.returncode, r.stdout, r.stderr[-2000:])


def test_no_device_means_an_error_status_not_a_fallback():
    """On a box without a GPU the compute entry points return PI_ERR_CUDA and a message naming the failed launch: there is
    no CPU path behind the C ABI."""
    import ctypes as C
    import pytest
    torch = pytest.importorskip("torch")
    if torch.cuda.is_available():
        pytest.skip("a device is present")
    from powerinfer_b200 import _lib
    lib = _lib.lib
    buf = (C.c_char * (1 << 20))()
    addr = (C.addressof(buf) + 255) & ~255
    rc = lib.pi_mul_mat(_lib.PI_TYPE_F16, addr, 8, 256, addr, 1, None, addr, addr, 1 << 19, None)
    assert rc == 2 and b"CUDA error" in lib.pi_last_error()
    rc = lib.pi_norm(addr, 1, 256, 1, C.c_float(1e-5), None, None, addr, None)
    assert rc == 2 and b"CUDA error" in lib.pi_last_error()
    assert not bytes(buf[:4096]).strip(b"\0")                      # nothing was computed on the host
