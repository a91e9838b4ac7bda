"""Wire contract: struct sizes, enumerator values and header hygiene of include/*.h."""
from __future__ import annotations

import os
import re
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
INC = ROOT / "include"
# where a checkout of the reference lives, if anywhere (the comparison with its headers is skipped without one)
REFERENCE = Path(os.environ.get("HTP_OPS_REFERENCE_DIR", "/nonexistent"))

PROBE = r"""
#include <stdio.h>
#include "op_reg.h"
#include "message.h"
%s
int main(void) {
  printf("%%zu %%zu %%zu %%zu ", sizeof(struct RpcmemBufAddr), sizeof(struct RmsNormF32Params),
         sizeof(struct MatMulParams), sizeof(struct FlashAttnParams));
  printf("%%zu %%zu %%zu %%zu %%zu ", sizeof(struct MessageState), sizeof(struct MessageHeader),
         sizeof(struct RequestHeader), sizeof(struct RpcmemMapRequest), sizeof(struct OpComputeRequest));
  printf("%%d %%d %%d %%d %%d %%d ", HTP_OPS_RMS_NORM_F32, HTP_OPS_MAT_MUL_PERMUTED_W16A32,
         HTP_OPS_MAT_MUL_PERMUTED_W4D16A32, HTP_OPS_MAT_MUL_PERMUTED_W8D16A32,
         HTP_OPS_MAT_MUL_PERMUTED_W4D16A32_IQ4_NL, HTP_OPS_FLASH_ATTN_QO_F32_KV_F16);
  printf("%%d %%d %%d ", REQUEST_TYPE_NO_OP, REQUEST_TYPE_RPCMEM_MAP, REQUEST_TYPE_OP_COMPUTE);
  printf("%%zu %%zu %%zu %%zu\n", sizeof(block_q4_0), sizeof(my_block_q4_0), sizeof(block_q8_0), sizeof(my_block_q8_0));
  return 0;
}
"""

EXPECTED = "8 24 36 60 8 16 8 8 4 0 1 2 3 4 5 0 1 2 18 144 34 272"


def _run_probe(tmp_path, include_dir: Path, quants_include: str, extra_flags=()):
    src = tmp_path / "probe.c"
    src.write_text(PROBE % quants_include)
    exe = tmp_path / "probe"
    subprocess.run(["gcc", "-std=gnu11", *extra_flags, "-I", str(include_dir), str(src), "-o", str(exe)], check=True)
    return subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.strip()


def test_struct_sizes_and_enum_values(tmp_path):
    assert _run_probe(tmp_path, INC, '#include "quants.h"') == EXPECTED


@pytest.mark.skipif(not REFERENCE.exists(), reason="the reference tree is only mounted in the build container")
def test_same_layout_as_reference_headers(tmp_path):
    """The reference's own op_reg.h / message.h / quants.h, compiled by the same probe, give the
    same sizes and values (its quants.h needs __fp16, spelled _Float16 on x86 gcc)."""
    got = _run_probe(tmp_path, REFERENCE / "include", '#include "dsp/quants.h"', ("-D__fp16=_Float16",))
    assert got == EXPECTED


def test_appended_ops_do_not_move_reference_indices(pkg):
    assert pkg.HTP_OPS_MAT_MUL_W4D16A16 == 6 and pkg.HTP_OPS_MAT_MUL_W8D16A16 == 7 and pkg.HTP_OPS_COUNT == 8
    text = (INC / "op_reg.h").read_text()
    assert "HTP_OPS_REFERENCE_COUNT 6" in text


def test_headers_compile_as_c_and_cxx(tmp_path):
    hdrs = ["op_reg.h", "message.h", "quants.h", "htp_ops_b200.h", "htp_ops.h", "host/session.h", "host/op_export.h",
            "host/buffers.h", "dsp/op_executor.h"]
    src = "".join(f'#include "{h}"\n' for h in hdrs) + "int main(void){return 0;}\n"
    (tmp_path / "a.c").write_text(src)
    (tmp_path / "a.cpp").write_text(src)
    subprocess.run(["gcc", "-std=gnu11", "-Wall", "-I", str(INC), str(tmp_path / "a.c"), "-o", str(tmp_path / "a")],
                   check=True)
    subprocess.run(["g++", "-std=c++17", "-Wall", "-I", str(INC), str(tmp_path / "a.cpp"), "-o", str(tmp_path / "b")],
                   check=True)


def _declared_functions():
    names = set()
    for h in INC.rglob("*.h"):
        text = re.sub(r"/\*.*?\*/", "", h.read_text(), flags=re.S)
        text = re.sub(r"//[^\n]*", "", text)
        text = re.sub(r"static inline[^{;]*\{.*?\n\}", "", text, flags=re.S)
        for m in re.finditer(r"\b([A-Za-z_][A-Za-z0-9_]*)\s*\([^;{}()]*\)\s*;", text):
            if m.group(1) not in ("static_assert", "_Static_assert", "__attribute__", "sizeof", "defined"):
                names.add(m.group(1))
    return names


def test_library_exports_every_declared_symbol(pkg, lib):
    declared = _declared_functions()
    assert {"htp_b200_mul_mat", "execute_op_simple", "open_dsp_session", "htp_buf_alloc",
            "htp_ops_create_channel"} <= declared
    missing = [n for n in sorted(declared) if not hasattr(lib, n)]
    assert not missing, f"declared in include/ but not exported: {missing}"
    assert declared <= set(pkg.EXPORTS), f"python binding table lacks {sorted(declared - set(pkg.EXPORTS))}"


def test_no_cpu_fallback(lib):
    """Without a CUDA device the session cannot be opened and compute entry points fail loudly."""
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    assert lib.open_dsp_session(0, 1) == -1
    assert lib.get_global_handle() == 2**64 - 1
    assert lib.htp_buf_alloc(1024) == -1
    assert lib.execute_op_simple(None) == -1
    assert lib.htp_b200_weight_bytes(2, 4096, 4096) == 9437184
    assert lib.htp_b200_weight_bytes(8, 4096, 11008) == 47906816
    assert lib.htp_b200_weight_bytes(8, 4096, 128256) == 558170112
    assert lib.htp_b200_weight_bytes(3, 4096, 32) == 0 and lib.htp_b200_weight_bytes(2, 100, 32) == 0
