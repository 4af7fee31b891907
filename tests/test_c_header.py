"""The drop-in boundary is a C header: it must compile as plain C (C99, warnings as errors), a C
program must link against the shared library and run without a GPU for the calls that need none, and
the layouts the C compiler gives the descriptor structs must be the ones the ctypes binding declares
(size and the offset of every field)."""
import ctypes
import shutil
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))

STRUCTS = {"pitch_buffer": "Buffer", "pitch_plane": "Plane", "pitch_append_src": "AppendSrc", "pitch_rope_bias": "RopeBias",
           "pitch_cache_desc": "CacheDesc", "pitch_cache_state": "CacheState", "pitch_attention_args": "AttentionArgs"}


@pytest.mark.skipif(shutil.which("gcc") is None, reason="no C compiler")
def test_header_compiles_as_c_links_and_matches_the_ctypes_layouts(tmp_path):
    from pitch_b200 import _native
    from pitch_b200.build import build
    lib = build()
    lines = ['#include <stddef.h>', '#include <stdio.h>', '#include "pitch_b200.h"', 'int main(void) {',
             '    printf("abi %d\\n", pitch_abi_version());', '    printf("stride %d\\n", pitch_code_stride(64, 3));',
             '    printf("status %s\\n", pitch_status_string(PITCH_ERR_INVALID_BIT_WIDTH));']
    for cname, pyname in STRUCTS.items():
        lines.append(f'    printf("{cname} size %zu\\n", sizeof({cname}));')
        for field, _ in getattr(_native, pyname)._fields_:
            lines.append(f'    printf("{cname} {field} %zu\\n", offsetof({cname}, {field}));')
    # every entry point of the header is a symbol the linker must find
    lines.append('    void* fns[] = {(void*)pitch_enqueue_encode, (void*)pitch_enqueue_decode, (void*)pitch_enqueue_channel_encode,'
                 ' (void*)pitch_enqueue_channel_decode, (void*)pitch_enqueue_rotate, (void*)pitch_enqueue_pack_codes,'
                 ' (void*)pitch_enqueue_unpack_codes, (void*)pitch_enqueue_cache_decode, (void*)pitch_enqueue_cache_append,'
                 ' (void*)pitch_enqueue_cache_step, (void*)pitch_enqueue_cache_newest, (void*)pitch_enqueue_cache_append_noalloc,'
                 ' (void*)pitch_cache_attention_workspace, (void*)pitch_enqueue_cache_attention, (void*)pitch_enqueue_rope_bias,'
                 ' (void*)pitch_enqueue_checksum, (void*)pitch_set_codebook, (void*)pitch_has_codebook, (void*)pitch_last_error};')
    lines += ['    printf("fns %d\\n", (int)(sizeof(fns) / sizeof(fns[0])));', '    return 0;', '}']
    src = tmp_path / "use.c"
    src.write_text("\n".join(lines) + "\n")
    exe = tmp_path / "use"
    cmd = ["gcc", "-std=c99", "-Wall", "-Wextra", "-Werror", "-Wno-pedantic", "-I", str(ROOT / "include"), str(src), "-o", str(exe),
           "-L", str(lib.parent), "-lpitch_b200", f"-Wl,-rpath,{lib.parent}"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    out = subprocess.run([str(exe)], capture_output=True, text=True, timeout=120)
    assert out.returncode == 0, out.stderr
    got = {}
    for line in out.stdout.splitlines():
        parts = line.split()
        got[" ".join(parts[:-1])] = parts[-1]
    assert int(got["abi"]) == _native.ABI_VERSION
    assert int(got["stride"]) == 24                                   # 64 codes of 3 bits: 6 words
    assert got["fns"] == "19"
    for cname, pyname in STRUCTS.items():
        S = getattr(_native, pyname)
        assert int(got[f"{cname} size"]) == ctypes.sizeof(S), cname
        for field, _ in S._fields_:
            assert int(got[f"{cname} {field}"]) == getattr(S, field).offset, (cname, field)
