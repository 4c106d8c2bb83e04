"""The C-ABI library loads without a GPU and exports every symbol the public header
declares, and argument validation fails cleanly before any launch."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "wuda_b200.h")


def declared_functions():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    names = re.findall(r"\b(wuda_[a-z0-9_]+)\s*\(", text)
    return sorted(set(names))


def test_header_declares_functions():
    names = declared_functions()
    assert "wuda_mqa_logits_fp8" in names and "wuda_last_error" in names


def test_library_exports_every_declared_symbol():
    import wuda_b200._lib as L
    for name in declared_functions():
        assert hasattr(L.lib, name), "libwuda_b200.so does not export %s" % name
    # and the ctypes table covers the header exactly
    assert sorted(L.SIGNATURES) == declared_functions()


def test_version_and_error_string():
    import wuda_b200._lib as L
    assert L.lib.wuda_version() >= 100
    assert isinstance(L.lib.wuda_last_error(), bytes)


def test_invalid_arguments_are_rejected_before_launch():
    import wuda_b200._lib as L
    vp = ctypes.c_void_p
    fake = vp(0x1000)
    # next_n = 3 is outside what the kernel implements
    st = L.lib.wuda_mqa_logits_fp8(fake, fake, fake, fake, fake, fake, 1, 3, 4, 64, 64 * 132, 4, 256, None, None)
    assert st == 2 and b"next_n" in L.lib.wuda_last_error()
    # page stride too small for the payload
    st = L.lib.wuda_mqa_logits_fp8(fake, fake, fake, fake, fake, fake, 1, 1, 4, 64, 64 * 128, 4, 256, None, None)
    assert st == 1 and b"page_stride_bytes" in L.lib.wuda_last_error()
    # bad page size
    st = L.lib.wuda_mqa_logits_fp8(fake, fake, fake, fake, fake, fake, 1, 1, 4, 48, 64 * 132, 4, 256, None, None)
    assert st == 1
    # NULL tensors
    st = L.lib.wuda_mqa_logits_fp8(None, fake, fake, fake, fake, fake, 1, 1, 4, 64, 64 * 132, 4, 256, None, None)
    assert st == 1 and b"NULL" in L.lib.wuda_last_error()
    # misaligned q
    st = L.lib.wuda_mqa_logits_fp8(vp(0x1004), fake, fake, fake, fake, fake, 1, 1, 4, 64, 64 * 132, 4, 256, None, None)
    assert st == 1 and b"aligned" in L.lib.wuda_last_error()
    # empty batch is a no-op
    assert L.lib.wuda_mqa_logits_fp8(None, None, None, None, None, None, 0, 1, 4, 64, 64 * 132, 4, 256, None, None) == 0


def test_struct_layouts_match_the_header(tmp_path):
    """The ctypes mirrors of the argument structs have the size and field offsets the C compiler
    gives the declarations in the header."""
    import subprocess
    import wuda_b200._lib as L
    structs = {"wuda_compressor_bundle": L.CompressorBundle, "wuda_window_bundle": L.WindowBundle,
               "wuda_cache_writers": L.CacheWriters, "wuda_csa_weights": L.CsaWeights, "wuda_csa_caches": L.CsaCaches,
               "wuda_csa_step": L.CsaStep, "wuda_csa_workspace": L.CsaWorkspace,
               "wuda_sparse_mla_args": L.SparseMlaArgs, "wuda_layer_weights": L.LayerWeights,
               "wuda_layer_state": L.LayerState, "wuda_layer_step": L.LayerStep}
    lines = ['#include <stdio.h>', '#include <stddef.h>', '#include "%s"' % HEADER, 'int main(void) {']
    for cname, cls in structs.items():
        lines.append('printf("%s %%zu\\n", sizeof(%s));' % (cname, cname))
        for field, _ in cls._fields_:
            lines.append('printf("%s.%s %%zu\\n", offsetof(%s, %s));' % (cname, field, cname, field))
    lines += ['return 0; }']
    src = tmp_path / "layout.c"
    src.write_text("\n".join(lines))
    exe = tmp_path / "layout"
    subprocess.check_call(["gcc", "-o", str(exe), str(src)])
    out = dict(line.split() for line in subprocess.check_output([str(exe)], text=True).splitlines())
    for cname, cls in structs.items():
        assert int(out[cname]) == ctypes.sizeof(cls), cname
        for field, _ in cls._fields_:
            assert int(out["%s.%s" % (cname, field)]) == getattr(cls, field).offset, "%s.%s" % (cname, field)


def test_benchmark_kinds_are_registered_and_documented():
    """Every kind the benchmark module documents in its header is registered, and the other way round."""
    import re
    from wuda_b200 import benchmarks
    documented = set(re.findall(r"wuda_b200\.benchmarks (\w+)", benchmarks.__doc__)) - {"one"}
    assert documented == set(benchmarks.KINDS), documented ^ set(benchmarks.KINDS)
    assert all(callable(f) for f in benchmarks.KINDS.values())


def test_the_documented_build_command_does_not_need_the_library():
    """`python -m wuda_b200.build` must be runnable on a tree whose library is missing or older than the ctypes table:
    the package's __init__ leaves the library alone for that one command (here: an up-to-date tree, so nothing is
    compiled; with the library's path pointed at a file that does not exist the import itself must still succeed)."""
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    code = ("import sys; sys.orig_argv = ['python', '-m', 'wuda_b200.build']; import wuda_b200; "
            "assert not hasattr(wuda_b200, 'lib'); print('ok')")
    out = subprocess.run([sys.executable, "-c", code], cwd=root, capture_output=True, text=True, timeout=300)
    assert out.returncode == 0 and out.stdout.strip() == "ok", out.stderr
    out = subprocess.run([sys.executable, "-m", "wuda_b200.build"], cwd=root, capture_output=True, text=True, timeout=1500)
    assert out.returncode == 0, out.stderr
