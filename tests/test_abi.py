"""The C-ABI library loads on a machine without a GPU and exports every symbol the public header declares."""
import ctypes as C

import eidola_b200 as eb
from eidola_b200 import capi


def test_header_symbols_are_exported():
    names = capi.declared_symbols()
    assert len(names) >= 30
    missing = [n for n in names if not hasattr(capi.lib(), n)]
    assert not missing, missing


def test_version_and_error_text():
    v = C.c_int32(0)
    capi.call("eb_version", C.byref(v))
    assert v.value == 5
    rc = capi.call_rc("eb_sched_create", C.c_int32(0), C.c_int32(16), C.c_int32(1), C.c_int32(1), C.c_uint64(0),
                      C.byref(C.c_void_p()))
    assert rc == -1
    assert "eb_sched_create" in capi.last_error()


def test_no_cpu_fallback_when_library_missing(tmp_path):
    import pytest
    with pytest.raises(ImportError, match="no CPU fallback"):
        capi.load_library(tmp_path / "libeidola_b200.so")


def test_validation_happens_before_any_launch():
    """Host validation errors are negative and need no device."""
    a = capi.AttnArgs()
    rc = capi.call_rc("eb_attn_paged_sink", C.byref(a), C.c_void_p())
    assert rc == -1 and "null" in capi.last_error()
    rc = capi.call_rc("eb_kv_append", C.c_void_p(16), C.c_int32(4), C.c_int32(8), C.c_int32(128), C.c_int32(16),
                      C.c_void_p(16), C.c_void_p(16), C.c_int64(512), C.c_void_p(16), C.c_int32(4), C.c_void_p(16),
                      C.c_void_p(16), C.c_int32(1), C.c_void_p())
    assert rc == -2 and "head_dim" in capi.last_error()


def test_oracle_config_mirror_matches_the_engine_binding():
    """The CPU checker declares eb_config on its own (so that it never imports the CUDA binding): same layout."""
    import ctypes as C

    from eidola_b200 import capi
    from oracle import binding as orc
    assert [(n, t) for n, t in capi.Config._fields_] == [(n, t) for n, t in orc.Config._fields_]
    assert C.sizeof(capi.Config) == C.sizeof(orc.Config)
    a, b = capi.make_config(n_layers=3, vocab=17), orc.make_config(n_layers=3, vocab=17)
    assert bytes(a) == bytes(b)


def test_a_plain_c_host_compiles_links_and_runs(tmp_path):
    """The headers are C (not only C++): a C11 host built with -pedantic links against the library and drives the
    entry points that need no device."""
    import shutil
    import subprocess
    from pathlib import Path
    root = Path(__file__).resolve().parent.parent
    gcc = shutil.which("gcc")
    assert gcc, "gcc is part of the image"
    lib = root / "eidola_b200" / "lib"
    exe = tmp_path / "c_host"
    subprocess.run([gcc, "-std=c11", "-Wall", "-Wextra", "-Werror", "-pedantic", "-I", str(root / "include"),
                    str(root / "tests" / "c_host" / "host.c"), "-L", str(lib), "-leidola_b200", "-Wl,-rpath," + str(lib), "-lm", "-o", str(exe)],
                   check=True, capture_output=True, text=True)
    r = subprocess.run([str(exe)], capture_output=True, text=True, timeout=60)
    assert r.returncode == 0, (r.returncode, r.stdout, r.stderr)
    assert "c host ok" in r.stdout and "0x3f80" in r.stdout
