"""The boundary is a plain C ABI: the header must compile as C11 and as C++17 without CUDA or
PyTorch headers, and a C program that only includes it must link against the library and run
(host-only entry points; nothing here needs a GPU)."""
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
HDR = ROOT / "include" / "metallic_cuda.h"
LIB_DIR = ROOT / "test-burn_b200"

C_PROGRAM = r'''
#include <stdio.h>
#include <string.h>
#include "metallic_cuda.h"

int main(void)
{
    /* the reference's #[repr(C)] parameter blocks, byte for byte */
    if (sizeof(KvPrepFusedParamsResolved) != 13 * 4) return 10;
    if (sizeof(SdpaParams) != 5 * 4) return 11;
    if (sizeof(SdpaPrefillParams) != 18 * 4) return 12;
    if (sizeof(SdpaPrefillSplitKParams) != 20 * 4) return 13;
    if (sizeof(RopeParamsResolved) != 4 * 4) return 14;
    if (sizeof(KvCacheWriteParamsResolved) != 7 * 4) return 15;
    if (mf_abi_version() == 0) return 1;
    if (strcmp(mf_status_name(MF_OK), "Ok") != 0) return 2;
    if (mf_align_capacity(2049) != 2176) return 3;             /* context.rs: round up to 128 */
    if (mf_grown_capacity(2048, 2049, 1u << 20) != 4096) return 4; /* x2 growth */
    if (mf_prefill_split_k(4096, 2048) != 8 || mf_prefill_split_k(2048, 16) != 4 || mf_prefill_split_k(512, 64) != 1)
        return 5;
    MfPagePool *pool = NULL;
    if (mf_page_pool_create(4, &pool) != MF_OK) return 6;
    uint32_t ids[4];
    if (mf_page_pool_alloc(pool, 3, ids) != MF_OK || mf_page_pool_free_count(pool) != 1) return 7;
    if (mf_page_pool_alloc(pool, 2, ids) != MF_ERR_OUT_OF_MEMORY) return 8;
    mf_page_pool_destroy(pool);
    /* a context cannot exist without a Blackwell GPU: the call must fail cleanly, not crash */
    MfContext *ctx = NULL;
    mf_status st = mf_context_create(0, NULL, &ctx);
    if (st == MF_OK) mf_context_destroy(ctx);
    printf("abi %u ok\n", mf_abi_version());
    return 0;
}
'''


def _run(cmd, **kw):
    return subprocess.run(cmd, capture_output=True, text=True, **kw)


def test_header_is_plain_c_and_cxx(tmp_path):
    c = tmp_path / "inc.c"
    c.write_text('#include "metallic_cuda.h"\nint main(void) { return 0; }\n')
    r = _run(["gcc", "-std=c11", "-Wall", "-Wextra", "-Werror", "-fsyntax-only", f"-I{HDR.parent}", str(c)])
    assert r.returncode == 0, r.stderr
    cxx = tmp_path / "inc.cpp"
    cxx.write_text('#include "metallic_cuda.h"\nint main() { return 0; }\n')
    r = _run(["g++", "-std=c++17", "-Wall", "-Wextra", "-Werror", "-fsyntax-only", f"-I{HDR.parent}", str(cxx)])
    assert r.returncode == 0, r.stderr


def test_c_program_links_and_runs(tmp_path):
    if not (LIB_DIR / "libmetallic_cuda.so").exists():
        pytest.fail("libmetallic_cuda.so is missing: run test-burn_b200/build.py")
    src = tmp_path / "abi.c"
    src.write_text(C_PROGRAM)
    exe = tmp_path / "abi"
    r = _run(["gcc", "-std=c11", "-Wall", "-Werror", f"-I{HDR.parent}", str(src), "-o", str(exe), f"-L{LIB_DIR}",
              "-lmetallic_cuda", f"-Wl,-rpath,{LIB_DIR}"])
    assert r.returncode == 0, r.stderr
    r = _run([str(exe)])
    assert r.returncode == 0, (r.returncode, r.stdout, r.stderr)
    assert "ok" in r.stdout
