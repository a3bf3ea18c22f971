"""CPU tests of the boundary: the C-ABI library loads and exports every symbol the header declares."""
import ctypes
import os
import re

import hyprstream_b200
from hyprstream_b200 import ffi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def header_functions():
    names = []
    for f in sorted(os.listdir(os.path.join(ROOT, "include"))):
        text = open(os.path.join(ROOT, "include", f)).read()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        names += re.findall(r"\b(hs_[a-z0-9_]+)\s*\(", text)
    return sorted(set(names))


def test_library_exports_every_declared_symbol():
    declared = header_functions()
    assert len(declared) >= 10
    for name in declared:
        assert hasattr(ffi.lib, name), f"{name} is declared in include/ but not exported"
    assert sorted(ffi.exported_symbols()) == declared, "ffi.py binds a different set than the header declares"


def test_version_and_struct_layout():
    assert ffi.lib.hs_attn_version() >= 100
    assert ctypes.sizeof(ffi.KVView) == 8 * 4 + 4 * 8  # matches struct hs_kv_view


def test_no_cpu_fallback_without_device():
    """Without a usable sm_100 device every compute entry point reports HS_ERR_DEVICE instead of computing."""
    import torch

    if torch.cuda.is_available():
        return
    st = ffi.lib.hs_quantize_blockwise(ffi.KV_INT8, None, ffi.DTYPE_BF16, 64, 64, ffi.SCALE_F32, None, None, None)
    assert st == ffi.HS_ERR_DEVICE and "device" in ffi.last_error().lower()


def test_rust_bindings_are_in_step_with_the_header():
    """crates/hyprstream-attn-sys/src/bindings.rs is generated from include/hs_attn.h: it must be current and name every
    exported entry point."""
    import os
    import re
    import subprocess
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    gen = os.path.join(root, "crates", "hyprstream-attn-sys", "gen_bindings.py")
    assert subprocess.run([sys.executable, gen, "--check"]).returncode == 0, "run crates/hyprstream-attn-sys/gen_bindings.py"
    text = open(os.path.join(root, "crates", "hyprstream-attn-sys", "src", "bindings.rs")).read()
    declared = set(re.findall(r"pub fn (hs_\w+)\(", text))
    from hyprstream_b200 import ffi

    assert declared == set(ffi.exported_symbols())


def test_ctypes_struct_layouts_match_the_header(tmp_path):
    """sizeof and the offset of the last field of every struct in include/hs_attn.h, as gcc sees them, against the ctypes
    mirrors in hyprstream_b200/ffi.py."""
    import subprocess

    structs = {"hs_kv_view": (ffi.KVView, "v_scale_pages"), "hs_gdn_layer_params": (ffi.GdnLayerParams, "kernel_size"),
               "hs_gdn_layer_io": (ffi.GdnLayerIO, "y"), "hs_qwen_attn_params": (ffi.QwenAttnParams, "softmax_scale"),
               "hs_qwen_attn_io": (ffi.QwenAttnIO, "out"), "hs_sched_plan": (ffi.SchedPlan, "n_running"),
               "hs_sched_stats_t": (ffi.SchedStats, "n_steps")}
    src = tmp_path / "layout.c"
    lines = ['#include <stdio.h>', '#include <stddef.h>', f'#include "{os.path.join(ROOT, "include", "hs_attn.h")}"', "int main(void) {"]
    for name, (_, last) in structs.items():
        lines.append(f'    printf("{name} %zu %zu\\n", sizeof({name}), offsetof({name}, {last}));')
    lines += ["    return 0;", "}"]
    src.write_text("\n".join(lines))
    exe = tmp_path / "layout"
    subprocess.check_call(["gcc", "-std=c99", "-o", str(exe), str(src)])
    for line in subprocess.check_output([str(exe)], text=True).splitlines():
        name, size, off = line.split()
        cls, last = structs[name]
        assert ctypes.sizeof(cls) == int(size), name
        assert getattr(cls, last).offset == int(off), name
