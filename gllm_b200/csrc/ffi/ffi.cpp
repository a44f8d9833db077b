// C ABI shim: embeds (or joins) the CPython runtime and drives gllm_b200.ffi_bridge.
#include <Python.h>

#include <cstdlib>
#include <cstring>
#include <mutex>
#include <string>

#include "gllm.h"

struct gllm_client {
  PyObject* obj;
};

static std::string g_init_error;
static std::once_flag g_once;
static bool g_we_initialised = false;

static void ensure_python() {
  std::call_once(g_once, [] {
    if (!Py_IsInitialized()) {
      Py_InitializeEx(0);
      g_we_initialised = true;
      PyEval_SaveThread();  // release the GIL; every entry point re-acquires it
    }
  });
}

static std::string py_error() {
  PyObject *t = nullptr, *v = nullptr, *tb = nullptr;
  PyErr_Fetch(&t, &v, &tb);
  PyErr_NormalizeException(&t, &v, &tb);
  std::string msg = "unknown error";
  if (v) {
    PyObject* s = PyObject_Str(v);
    if (s) {
      const char* c = PyUnicode_AsUTF8(s);
      if (c) msg = c;
      Py_DECREF(s);
    }
  }
  Py_XDECREF(t);
  Py_XDECREF(v);
  Py_XDECREF(tb);
  return msg;
}

static char* dup_str(const std::string& s) {
  char* p = static_cast<char*>(std::malloc(s.size() + 1));
  std::memcpy(p, s.c_str(), s.size() + 1);
  return p;
}

extern "C" {

__attribute__((visibility("default"))) const char* gllm_client_version(void) { return "gllm_b200 0.1.0"; }
__attribute__((visibility("default"))) const char* gllm_last_init_error(void) { return g_init_error.c_str(); }

__attribute__((visibility("default"))) gllm_client* gllm_init(const char* model_id, const char* options_json) {
  ensure_python();
  PyGILState_STATE gil = PyGILState_Ensure();
  gllm_client* out = nullptr;
  PyObject* mod = PyImport_ImportModule("gllm_b200.ffi_bridge");
  if (!mod) {
    g_init_error = "import gllm_b200.ffi_bridge failed: " + py_error();
  } else {
    PyObject* obj = PyObject_CallMethod(mod, "create", "ss", model_id ? model_id : "", options_json ? options_json : "");
    if (!obj) {
      g_init_error = py_error();
    } else {
      out = new gllm_client{obj};
      g_init_error.clear();
    }
    Py_DECREF(mod);
  }
  PyGILState_Release(gil);
  return out;
}

__attribute__((visibility("default"))) void gllm_destroy(gllm_client* c) {
  if (!c) return;
  PyGILState_STATE gil = PyGILState_Ensure();
  PyObject* r = PyObject_CallMethod(c->obj, "close", nullptr);
  if (!r) PyErr_Clear();
  Py_XDECREF(r);
  Py_DECREF(c->obj);
  PyGILState_Release(gil);
  delete c;
}

__attribute__((visibility("default"))) gllm_generate_result* gllm_generate(gllm_client* c, const char* prompt,
                                                                            int max_tokens, float temperature,
                                                                            int top_k, float top_p) {
  auto* res = static_cast<gllm_generate_result*>(std::calloc(1, sizeof(gllm_generate_result)));
  if (!c || !prompt) {
    res->error = 1;
    res->error_message = dup_str("null client or prompt");
    return res;
  }
  PyGILState_STATE gil = PyGILState_Ensure();
  PyObject* r = PyObject_CallMethod(c->obj, "generate", "sifif", prompt, max_tokens, double(temperature), top_k,
                                    double(top_p));
  if (!r) {
    res->error = 2;
    res->error_message = dup_str(py_error());
  } else {
    // (text, [token ids], prompt_tokens, finish_reason)
    PyObject* text = PyTuple_GetItem(r, 0);
    PyObject* ids = PyTuple_GetItem(r, 1);
    const char* t = text ? PyUnicode_AsUTF8(text) : nullptr;
    res->text = dup_str(t ? t : "");
    const Py_ssize_t n = ids ? PyList_Size(ids) : 0;
    res->num_tokens = static_cast<int>(n);
    res->token_ids = static_cast<int*>(std::malloc(sizeof(int) * (n > 0 ? n : 1)));
    for (Py_ssize_t i = 0; i < n; ++i) res->token_ids[i] = static_cast<int>(PyLong_AsLong(PyList_GetItem(ids, i)));
    res->prompt_tokens = static_cast<int>(PyLong_AsLong(PyTuple_GetItem(r, 2)));
    res->finish_reason = static_cast<int>(PyLong_AsLong(PyTuple_GetItem(r, 3)));
    Py_DECREF(r);
  }
  PyGILState_Release(gil);
  return res;
}

__attribute__((visibility("default"))) void gllm_free_generate_result(gllm_generate_result* r) {
  if (!r) return;
  std::free(r->text);
  std::free(r->token_ids);
  std::free(r->error_message);
  std::free(r);
}

}  // extern "C"
