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


class Result(ctypes.Structure):        # the reference's GllmGenerateResult {text, error}, returned by value
    _fields_ = [("text", ctypes.c_char_p), ("error", ctypes.c_char_p)]


class ResultEx(ctypes.Structure):
    _fields_ = [("text", ctypes.c_char_p), ("token_ids", ctypes.POINTER(ctypes.c_int)), ("num_tokens", ctypes.c_int),
                ("prompt_tokens", ctypes.c_int), ("finish_reason", ctypes.c_int), ("error", ctypes.c_int),
                ("error_message", ctypes.c_char_p)]


OPTS = b'{"device": "cpu", "dtype": "fp32", "max_num_seqs": 2, "max_model_len": 128, "max_batch_tokens": 64}'


def _load():
    L = ctypes.PyDLL(str(LIB))          # PyDLL: the calling thread keeps the GIL; the shim's Ensure() nests
    u32, i32, f32, vp, cp = ctypes.c_uint32, ctypes.c_int32, ctypes.c_float, ctypes.c_void_p, ctypes.c_char_p
    L.gllm_init.restype = vp
    L.gllm_init.argtypes = [cp, u32]
    L.gllm_init_with_options.restype = vp
    L.gllm_init_with_options.argtypes = [cp, u32, cp]
    L.gllm_generate.restype = Result
    L.gllm_generate.argtypes = [vp, cp, u32, f32, u32, f32, i32]
    L.gllm_free_generate_result.argtypes = [ctypes.POINTER(Result)]
    L.gllm_generate_ex.restype = ctypes.POINTER(ResultEx)
    L.gllm_generate_ex.argtypes = [vp, cp, u32, f32, u32, f32, i32]
    L.gllm_free_generate_result_ex.argtypes = [ctypes.POINTER(ResultEx)]
    L.gllm_destroy.argtypes = [vp]
    L.gllm_client_version.restype = cp
    L.gllm_last_init_error.restype = cp
    L.gllm_embed.restype = ctypes.c_int
    L.gllm_embed.argtypes = [vp, cp, ctypes.POINTER(ctypes.c_float), ctypes.c_int]
    return L


def test_c_abi_reference_signatures_in_process(monkeypatch):
    """gllm_init(model_id, kind) / gllm_generate(..., thinking_budget) -> {text, error} by value, as in src/ffi.rs."""
    L = _load()
    assert L.gllm_client_version().startswith(b"gllm_b200")
    monkeypatch.setenv("GLLM_FFI_OPTIONS", OPTS.decode())
    h = L.gllm_init(b"tiny-llama", 0)
    assert h, L.gllm_last_init_error()
    r = L.gllm_generate(h, b"hello world", 5, 0.0, 0, 1.0, 0)
    assert r.error is None and r.text is not None
    r2 = L.gllm_generate(h, b"hello world", 5, 0.0, 0, 1.0, -1)
    assert r2.text == r.text
    L.gllm_free_generate_result(ctypes.byref(r)); L.gllm_free_generate_result(ctypes.byref(r2))
    assert r.text is None and r.error is None            # the strings are freed and the pointers cleared
    bad = L.gllm_generate(None, b"x", 1, 0.0, 0, 1.0, 0)
    assert bad.text is None and b"null pointer" in bad.error
    L.gllm_free_generate_result(ctypes.byref(bad))
    L.gllm_destroy(h)
    assert not L.gllm_init(b"/nonexistent/model/dir", 0) and L.gllm_last_init_error()
    assert not L.gllm_init(None, 0)


def test_c_abi_extended_entry_points_in_process():
    L = _load()
    h = L.gllm_init_with_options(b"tiny-llama", 0, OPTS)
    assert h, L.gllm_last_init_error()
    r = L.gllm_generate_ex(h, b"hello world", 5, 0.0, 0, 1.0, 0)
    assert r.contents.error == 0 and 1 <= r.contents.num_tokens <= 5 and r.contents.prompt_tokens == 11
    ids = [r.contents.token_ids[i] for i in range(r.contents.num_tokens)]
    r2 = L.gllm_generate_ex(h, b"hello world", 5, 0.0, 0, 1.0, 0)
    assert ids == [r2.contents.token_ids[i] for i in range(r2.contents.num_tokens)]
    L.gllm_free_generate_result_ex(r); L.gllm_free_generate_result_ex(r2)
    bad = L.gllm_generate_ex(None, b"x", 1, 0.0, 0, 1.0, 0)
    assert bad.contents.error == 1
    L.gllm_free_generate_result_ex(bad)
    L.gllm_destroy(h)
    # kind = 1 opens an embedding model through the same ABI
    e = L.gllm_init_with_options(b"tiny-bert", 1, b'{"device": "cpu", "dtype": "fp32"}')
    assert e, L.gllm_last_init_error()
    buf = (ctypes.c_float * 256)()
    dim = L.gllm_embed(e, b"some text", buf, 256)
    assert dim == 128 and abs(sum(buf[i] * buf[i] for i in range(dim)) - 1.0) < 1e-3
    L.gllm_destroy(e)


@pytest.mark.skipif(shutil.which("gcc") is None, reason="no C compiler")
def test_c_abi_from_a_c_program(tmp_path):
    src = tmp_path / "main.c"
    src.write_text('''
#include <stdio.h>
#include "gllm.h"
int main(void) {
  /* the reference's own call sequence: init(model, kind) -> generate(..., thinking_budget) -> free -> destroy */
  GllmContext* c = gllm_init("tiny-llama", 0);
  if (!c) { printf("INIT_FAILED %s\\n", gllm_last_init_error()); return 1; }
  GllmGenerateResult r = gllm_generate(c, "hello", 4, 0.0f, 0, 1.0f, 0);
  printf("TEXT %s ERR %s\\n", r.text ? "yes" : "no", r.error ? r.error : "none");
  gllm_free_generate_result(&r);
  GllmGenerateResultEx* x = gllm_generate_ex(c, "hello", 4, 0.0f, 0, 1.0f, 0);
  printf("TOKENS %d ERR %d PROMPT %d\\n", x->num_tokens, x->error, x->prompt_tokens);
  gllm_free_generate_result_ex(x);
  gllm_destroy(c);
  return 0;
}''')
    exe = tmp_path / "main"
    inc = ROOT / "gllm_b200" / "csrc" / "ffi"
    subprocess.run(["gcc", str(src), "-I", str(inc), "-L", str(LIB.parent), "-lgllm_ffi", f"-Wl,-rpath,{LIB.parent}", "-o", str(exe)], check=True)
    env = dict(os.environ, PYTHONPATH=str(ROOT), PYTHONHOME=sys.base_prefix, GLLM_FFI_OPTIONS=OPTS.decode())
    site = [p for p in sys.path if p.endswith("site-packages")]
    env["PYTHONPATH"] = os.pathsep.join([str(ROOT)] + site)
    r = subprocess.run([str(exe)], env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "ERR 0 PROMPT 5" in r.stdout and "TEXT yes ERR none" in r.stdout, r.stdout + r.stderr
