"""The public header is plain C: a C translation unit that includes it compiles with gcc -std=c99 -pedantic,
links against the shared library and can call the identity functions without a GPU."""
import shutil
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent

PROGRAM = r"""
#include <stdio.h>
#include <string.h>
#include "axiom_b200.h"
#include "axiom_b200_engine.h"

int main(void) {
    axiom_abi_info info;
    axiom_config cfg;
    axiom_qk_rope_args args;
    axiom_rope_config rope;
    memset(&info, 0, sizeof info);
    memset(&cfg, 0, sizeof cfg);
    memset(&args, 0, sizeof args);
    memset(&rope, 0, sizeof rope);
    info.abi_version = AXIOM_ABI_VERSION;
    if (axiom_abi_version() != AXIOM_ABI_VERSION) return 1;
    if (axiom_abi_check(AXIOM_ABI_VERSION) != AXIOM_OK) return 2;
    if (axiom_abi_info_get(&info) != AXIOM_OK || strcmp(info.backend, "cuda") != 0) return 3;
    if (strcmp(axiom_status_string(AXIOM_ERR_BUDGET), "budget exceeded") != 0) return 4;
    if (axiom_nvfp4_scale_plane_bytes(4096u, 320u, AXIOM_SCALE_LAYOUT_TILED) != 32u * 80u * 512u) return 5;
    /* argument checks come before any device work */
    if (axiom_qwen38_fused_qk_norm_rope_paged_bf16_device(0, &args, NULL) != AXIOM_ERR_INVALID_ARGUMENT) return 6;
    if (axiom_qwen38_fused_swiglu_fp8_bf16_device(0, NULL, 1u, 8u, NULL, NULL, NULL) != AXIOM_ERR_INVALID_ARGUMENT) return 7;
    {
        axiom_engine_seq seq;
        axiom_b200_step_provider *provider = NULL;
        memset(&seq, 0, sizeof seq);
        if (axiom_b200_step_provider_create(NULL, NULL, &provider) != AXIOM_ERR_INVALID_ARGUMENT || provider != NULL) return 8;
        if (axiom_b200_step_provider_forward_step(NULL, NULL, 0, NULL) != AXIOM_ERR_INVALID_ARGUMENT) return 9;
    }
    printf("%s\n", axiom_version());
    return 0;
}
"""


def test_header_is_c_and_links(axk, tmp_path):
    gcc = "/usr/bin/gcc" if Path("/usr/bin/gcc").exists() else shutil.which("gcc")
    if not gcc:
        pytest.skip("no C compiler")
    src = tmp_path / "link_check.c"
    src.write_text(PROGRAM)
    exe = tmp_path / "link_check"
    lib_dir = Path(axk.LIB_PATH).parent
    cmd = [gcc, "-std=c99", "-pedantic", "-Wall", "-Werror", f"-I{ROOT / 'include'}", str(src), "-o", str(exe),
           f"-L{lib_dir}", "-laxiom_b200", f"-Wl,-rpath,{lib_dir}"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    assert res.returncode == 0, res.stderr
    run = subprocess.run([str(exe)], capture_output=True, text=True)
    assert run.returncode == 0, (run.returncode, run.stderr)
    assert "sm_100a" in run.stdout
