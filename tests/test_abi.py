"""CPU checks of the C-ABI boundary: the shared library loads, exports every symbol declared
in include/nlh_ffi.h with a consistent prototype table, and the drop-in names match the
reference's extern "C" block (no compute is launched here)."""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

# the subset of core/src/cuda_ffi.rs on the hot path (names only; signatures are in the header)
REFERENCE_SYMBOLS = """
swa_forward_f32_cuda swa_backward_f32_cuda
delta_forward_f32_cuda delta_backward_f32_cuda titans_forward_f32_cuda titans_backward_f32_cuda
hebbian_forward_f32_cuda hebbian_backward_f32_cuda
delta_forward_ckpt_f32_cuda titans_forward_ckpt_f32_cuda hebbian_forward_ckpt_f32_cuda
delta_backward_segment_f32_cuda titans_backward_segment_f32_cuda hebbian_backward_segment_f32_cuda
dgd_forward_f32_cuda dgd_backward_f32_cuda dgd_forward_ckpt_f32_cuda dgd_backward_segment_f32_cuda
delta_chunkwise_forward_f32_cuda delta_chunkwise_backward_f32_cuda
titans_chunkwise_forward_f32_cuda titans_chunkwise_backward_f32_cuda
error_subtract_clip_f32_cuda delta_phase2_forward_f32_cuda titans_phase2_forward_f32_cuda
delta_phase2_backward_f32_cuda titans_phase2_backward_f32_cuda
m_norm_clamp_f32_cuda m_norm_clamp_batch_f32_cuda
adamw_update_cuda grad_norm_sq_cuda dot_product_partial_f32_cuda grad_scale_cuda
reduce_partials_clip_cuda grad_scale_conditional_cuda
dgd_fused_forward_f32_cuda titans_fused_forward_f32_cuda
""".split()


@pytest.fixture(scope="module")
def built():
    from nl_hecate_b200 import build
    return build.build()


def test_library_exports_every_header_symbol(built):
    from nl_hecate_b200 import ffi
    protos = ffi.parse_header()
    assert len(protos) >= 45
    handle = C.CDLL(built)
    for name in protos:
        assert hasattr(handle, name), f"{name} declared in include/nlh_ffi.h but not exported"
    lib = ffi.lib()
    assert lib.nlh_abi_version() == 1
    assert lib.nlh_last_status() == 0 and lib.nlh_last_error() == b""


def test_reference_drop_in_names_present(built):
    from nl_hecate_b200 import ffi
    protos = ffi.parse_header()
    for name in REFERENCE_SYMBOLS:
        assert name in protos, name


def test_drop_in_arity_matches_reference_ffi():
    """Argument counts of a few entries, read off core/src/cuda_ffi.rs (lines cited in the header)."""
    from nl_hecate_b200 import ffi
    protos = ffi.parse_header()
    arity = {"swa_forward_f32_cuda": 11, "swa_backward_f32_cuda": 14, "titans_forward_f32_cuda": 18,
             "titans_backward_f32_cuda": 21, "delta_forward_f32_cuda": 15,
             "hebbian_backward_f32_cuda": 13, "titans_chunkwise_backward_f32_cuda": 23,
             "titans_phase2_backward_f32_cuda": 26, "adamw_update_cuda": 12,
             "titans_fused_forward_f32_cuda": 28, "titans_backward_segment_f32_cuda": 25}
    for name, n in arity.items():
        assert len(protos[name][1]) == n, (name, len(protos[name][1]))
    assert protos["adamw_update_cuda"][0] is C.c_uint32      # cudaError_t
    assert protos["titans_forward_f32_cuda"][0] is None      # void


def test_desc_struct_layout_matches_header():
    from nl_hecate_b200 import ffi
    text = open(os.path.join(ROOT, "include", "nlh_ffi.h")).read()
    body = re.search(r"typedef struct nlh_adamw_tensor_desc \{(.*?)\}", text, re.S).group(1)
    body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
    fields = re.findall(r"(float|int32_t)\s+(\w+);", body)
    assert [f[1] for f in fields] == [f[0] for f in ffi.AdamWTensorDesc._fields_]
    assert C.sizeof(ffi.AdamWTensorDesc) == 32


def test_product_package_does_not_touch_the_oracle():
    pkg = os.path.join(ROOT, "nl_hecate_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                src = open(os.path.join(dirpath, f)).read()
                assert "import oracle" not in src and "from oracle" not in src, f
                assert "nlh_oracle" not in src, f


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    from nl_hecate_b200 import ffi
    monkeypatch.setattr(ffi, "_lib", None)
    monkeypatch.setattr(ffi, "LIB_PATH", str(tmp_path / "absent.so"))
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        ffi.lib()


def test_bench_reference_arm_prints_the_contract_line():
    """`bench.py --impl reference` (CPU arm, no GPU needed) prints one JSON line with the keys the
    measurement contract names; checked on the smallest workload so that it takes seconds."""
    import json
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = subprocess.run([sys.executable, os.path.join(root, "bench.py"), "--impl", "reference", "--workload",
                          "adamw", "--steps", "1", "--warmup", "0"], capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr[-500:]
    lines = [l for l in out.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1
    rec = json.loads(lines[0])
    for key in ("impl", "metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better",
                "scaling", "vs_baseline", "dtype", "data", "config", "cpu_baseline", "e2e"):
        assert key in rec, key
    assert rec["impl"] == "reference" and rec["value"] > 0
    assert rec["cpu_baseline"]["kind"] == "port" and rec["cpu_baseline"]["cores"] >= 1
    assert rec["e2e"]["h2d_bytes_per_step"] == 0 and rec["e2e"]["d2h_bytes_per_step"] == 0


def test_drop_in_prototypes_match_the_reference_declarations():
    """Every non-nlh_ prototype of include/nlh_ffi.h against the reference's Rust declaration of
    the same name (tests/golden/ffi_signatures.json, extracted from core/src/cuda_ffi.rs by
    tests/golden/make_ffi_signatures.py): same argument count, order, names and types, same
    return type."""
    import json
    import os
    import re
    here = os.path.dirname(os.path.abspath(__file__))
    sigs = json.load(open(os.path.join(here, "golden", "ffi_signatures.json")))
    hdr = open(os.path.join(os.path.dirname(here), "include", "nlh_ffi.h")).read()
    hdr = re.sub(r"/\*.*?\*/", "", hdr, flags=re.S)
    tmap = {"*const f32": "const float*", "*mut f32": "float*", "*const u16": "const uint16_t*",
            "*mut u16": "uint16_t*", "i32": "int32_t", "f32": "float", "*const i32": "const int32_t*",
            "*mut i32": "int32_t*", "u32": "uint32_t", "i64": "int64_t"}
    rmap = {None: "void", "u32": "uint32_t", "i32": "int32_t"}
    checked = 0
    for m in re.finditer(r"^(void|int32_t|uint32_t)\s+(\w+)\s*\((.*?)\)\s*;", hdr, flags=re.S | re.M):
        ret, name, args = m.group(1), m.group(2), m.group(3)
        if name.startswith("nlh_"):
            continue
        assert name in sigs, f"{name} is not declared by the reference"
        want = sigs[name]
        got = []
        for a in args.split(","):
            mm = re.match(r"(.*?)(\w+)$", " ".join(a.split()))
            got.append((mm.group(2), mm.group(1).strip().replace(" *", "*").replace(" ", "")))
        exp = [(n, tmap[t].replace(" ", "")) for n, t in want["args"]]
        assert got == exp, (name, got, exp)
        assert rmap[want["ret"]] == ret, name
        checked += 1
    assert checked >= 40
