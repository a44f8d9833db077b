"""The C ABI, called through ctypes from inside a Python process (the shim joins the running interpreter) and
from a standalone C program when a C compiler is present."""
import ctypes
import os
import shutil
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
LIB = ROOT / "gllm_b200" / "_lib" / "libgllm_ffi.so"


class Result(ctypes.Structure):
    _fields_ = [("text", ctypes.c_char_p), ("token_ids", ctypes.POINTER(ctypes.c_int)), ("num_tokens", ctypes.c_int),
                ("prompt_tokens", ctypes.c_int), ("finish_reason", ctypes.c_int), ("error", ctypes.c_int),
                ("error_message", ctypes.c_char_p)]


def _load():
    L = ctypes.PyDLL(str(LIB))          # PyDLL: the calling thread keeps the GIL; the shim's Ensure() nests
    L.gllm_init.restype = ctypes.c_void_p
    L.gllm_init.argtypes = [ctypes.c_char_p, ctypes.c_char_p]
    L.gllm_generate.restype = ctypes.POINTER(Result)
    L.gllm_generate.argtypes = [ctypes.c_void_p, ctypes.c_char_p, ctypes.c_int, ctypes.c_float, ctypes.c_int, ctypes.c_float]
    L.gllm_free_generate_result.argtypes = [ctypes.POINTER(Result)]
    L.gllm_destroy.argtypes = [ctypes.c_void_p]
    L.gllm_client_version.restype = ctypes.c_char_p
    L.gllm_last_init_error.restype = ctypes.c_char_p
    return L


def test_c_abi_in_process():
    L = _load()
    assert L.gllm_client_version().startswith(b"gllm_b200")
    h = L.gllm_init(b"tiny-llama", b'{"device": "cpu", "dtype": "fp32", "max_num_seqs": 2, "max_model_len": 128, "max_batch_tokens": 64}')
    assert h, L.gllm_last_init_error()
    r = L.gllm_generate(h, b"hello world", 5, 0.0, 0, 1.0)
    assert r.contents.error == 0 and 1 <= r.contents.num_tokens <= 5 and r.contents.prompt_tokens == 11
    ids = [r.contents.token_ids[i] for i in range(r.contents.num_tokens)]
    r2 = L.gllm_generate(h, b"hello world", 5, 0.0, 0, 1.0)
    assert ids == [r2.contents.token_ids[i] for i in range(r2.contents.num_tokens)]
    L.gllm_free_generate_result(r); L.gllm_free_generate_result(r2)
    bad = L.gllm_generate(None, b"x", 1, 0.0, 0, 1.0)
    assert bad.contents.error == 1
    L.gllm_free_generate_result(bad)
    L.gllm_destroy(h)
    assert not L.gllm_init(b"/nonexistent/model/dir", b"") and L.gllm_last_init_error()


@pytest.mark.skipif(shutil.which("gcc") is None, reason="no C compiler")
def test_c_abi_from_a_c_program(tmp_path):
    src = tmp_path / "main.c"
    src.write_text('''
#include <stdio.h>
#include "gllm.h"
int main(void) {
  gllm_client* c = gllm_init("tiny-llama", "{\\"device\\": \\"cpu\\", \\"dtype\\": \\"fp32\\", \\"max_num_seqs\\": 2, \\"max_model_len\\": 128, \\"max_batch_tokens\\": 64}");
  if (!c) { printf("INIT_FAILED %s\\n", gllm_last_init_error()); return 1; }
  gllm_generate_result* r = gllm_generate(c, "hello", 4, 0.0f, 0, 1.0f);
  printf("TOKENS %d ERR %d PROMPT %d\\n", r->num_tokens, r->error, r->prompt_tokens);
  gllm_free_generate_result(r);
  gllm_destroy(c);
  return 0;
}''')
    exe = tmp_path / "main"
    inc = ROOT / "gllm_b200" / "csrc" / "ffi"
    subprocess.run(["gcc", str(src), "-I", str(inc), "-L", str(LIB.parent), "-lgllm_ffi", f"-Wl,-rpath,{LIB.parent}", "-o", str(exe)], check=True)
    env = dict(os.environ, PYTHONPATH=str(ROOT), PYTHONHOME=sys.base_prefix)
    site = [p for p in sys.path if p.endswith("site-packages")]
    env["PYTHONPATH"] = os.pathsep.join([str(ROOT)] + site)
    r = subprocess.run([str(exe)], env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "ERR 0 PROMPT 5" in r.stdout, r.stdout + r.stderr
