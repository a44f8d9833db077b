// C ABI shim: embeds (or joins) the CPython runtime and drives gllm_b200.ffi_bridge.
#include <Python.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <string>

#include "gllm.h"

struct GllmContext {
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

#define GLLM_EXPORT __attribute__((visibility("default")))

static PyObject* call_generate(GllmContext* c, const char* prompt, uint32_t max_tokens, float temperature,
                               uint32_t top_k, float top_p, int32_t thinking_budget) {
  // -> (text, [token ids], prompt_tokens, finish_reason)
  return PyObject_CallMethod(c->obj, "generate", "sIfIfi", prompt, static_cast<unsigned int>(max_tokens),
                             double(temperature), static_cast<unsigned int>(top_k), double(top_p), int(thinking_budget));
}

extern "C" {

GLLM_EXPORT const char* gllm_client_version(void) { return "gllm_b200 0.2.0"; }
GLLM_EXPORT const char* gllm_last_init_error(void) { return g_init_error.c_str(); }

GLLM_EXPORT GllmContext* gllm_init_with_options(const char* model_id, uint32_t kind, const char* options_json) {
  if (!model_id) {
    g_init_error = "null model id";
    return nullptr;
  }
  ensure_python();
  PyGILState_STATE gil = PyGILState_Ensure();
  GllmContext* out = nullptr;
  PyObject* mod = PyImport_ImportModule("gllm_b200.ffi_bridge");
  if (!mod) {
    g_init_error = "import gllm_b200.ffi_bridge failed: " + py_error();
  } else {
    PyObject* obj = PyObject_CallMethod(mod, "create", "sIs", model_id, static_cast<unsigned int>(kind),
                                        options_json ? options_json : "");
    if (!obj) {
      g_init_error = py_error();
      fprintf(stderr, "[gllm FFI] init failed: %s\n", g_init_error.c_str());
    } else {
      out = new GllmContext{obj};
      g_init_error.clear();
    }
    Py_DECREF(mod);
  }
  PyGILState_Release(gil);
  return out;
}

// Reference signature: the options come from GLLM_FFI_OPTIONS (JSON) when set.
GLLM_EXPORT GllmContext* gllm_init(const char* model_id, uint32_t kind) {
  return gllm_init_with_options(model_id, kind, std::getenv("GLLM_FFI_OPTIONS"));
}

GLLM_EXPORT void gllm_destroy(GllmContext* c) {
  if (!c) return;
  PyGILState_STATE gil = PyGILState_Ensure();
  PyObject* r = PyObject_CallMethod(c->obj, "close", nullptr);
  if (!r) PyErr_Clear();
  Py_XDECREF(r);
  Py_DECREF(c->obj);
  PyGILState_Release(gil);
  delete c;
}

GLLM_EXPORT GllmGenerateResult gllm_generate(GllmContext* c, const char* prompt, uint32_t max_tokens, float temperature,
                                             uint32_t top_k, float top_p, int32_t thinking_budget) {
  GllmGenerateResult res = {nullptr, nullptr};
  if (!c || !prompt) {
    res.error = dup_str("null pointer argument");
    return res;
  }
  PyGILState_STATE gil = PyGILState_Ensure();
  PyObject* r = call_generate(c, prompt, max_tokens, temperature, top_k, top_p, thinking_budget);
  if (!r) {
    res.error = dup_str(py_error());
  } else {
    PyObject* text = PyTuple_GetItem(r, 0);
    const char* t = text ? PyUnicode_AsUTF8(text) : nullptr;
    res.text = dup_str(t ? t : "");
    Py_DECREF(r);
  }
  PyGILState_Release(gil);
  return res;
}

GLLM_EXPORT void gllm_free_generate_result(GllmGenerateResult* r) {
  if (!r) return;
  std::free(r->text);
  std::free(r->error);
  r->text = nullptr;
  r->error = nullptr;
}

GLLM_EXPORT GllmGenerateResultEx* gllm_generate_ex(GllmContext* c, const char* prompt, uint32_t max_tokens,
                                                   float temperature, uint32_t top_k, float top_p,
                                                   int32_t thinking_budget) {
  auto* res = static_cast<GllmGenerateResultEx*>(std::calloc(1, sizeof(GllmGenerateResultEx)));
  if (!c || !prompt) {
    res->error = 1;
    res->error_message = dup_str("null client or prompt");
    return res;
  }
  PyGILState_STATE gil = PyGILState_Ensure();
  PyObject* r = call_generate(c, prompt, max_tokens, temperature, top_k, top_p, thinking_budget);
  if (!r) {
    res->error = 2;
    res->error_message = dup_str(py_error());
  } else {
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

GLLM_EXPORT void gllm_free_generate_result_ex(GllmGenerateResultEx* r) {
  if (!r) return;
  std::free(r->text);
  std::free(r->token_ids);
  std::free(r->error_message);
  std::free(r);
}

GLLM_EXPORT int gllm_embed(GllmContext* c, const char* text, float* out, int capacity) {
  if (!c || !text || !out) return -1;
  PyGILState_STATE gil = PyGILState_Ensure();
  int dim = -1;
  PyObject* r = PyObject_CallMethod(c->obj, "embed", "s", text);
  if (!r) {
    g_init_error = py_error();
  } else {
    const Py_ssize_t n = PyList_Size(r);
    dim = static_cast<int>(n);
    for (Py_ssize_t i = 0; i < n && i < capacity; ++i) out[i] = static_cast<float>(PyFloat_AsDouble(PyList_GetItem(r, i)));
    Py_DECREF(r);
  }
  PyGILState_Release(gil);
  return dim;
}

GLLM_EXPORT int gllm_rerank_score(GllmContext* c, const char* query, const char* document, float* score) {
  if (!c || !query || !document || !score) return -1;
  PyGILState_STATE gil = PyGILState_Ensure();
  int rc = -1;
  PyObject* r = PyObject_CallMethod(c->obj, "rerank_score", "ss", query, document);
  if (!r) {
    g_init_error = py_error();
  } else {
    *score = static_cast<float>(PyFloat_AsDouble(r));
    rc = 0;
    Py_DECREF(r);
  }
  PyGILState_Release(gil);
  return rc;
}

}  // extern "C"
