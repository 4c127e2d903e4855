// C API implementation: a thin bridge from C calls to mythos_b200.capi (Python), see oil_c_api.h.
#include "oil_c_api.h"

#include <Python.h>

#include <cstdlib>
#include <cstring>
#include <mutex>
#include <string>

namespace {

thread_local std::string g_error;
std::once_flag g_init_once;
bool g_owns_interpreter = false;

void ensure_interpreter() {
  std::call_once(g_init_once, [] {
    if (!Py_IsInitialized()) {
      Py_InitializeEx(0);
      g_owns_interpreter = true;
      PyEval_SaveThread();  // release the lock taken by initialisation; calls re-acquire it
    }
  });
}

struct Gil {
  PyGILState_STATE st;
  Gil() { st = PyGILState_Ensure(); }
  ~Gil() { PyGILState_Release(st); }
};

void capture_python_error(const char* what) {
  PyObject *type = nullptr, *value = nullptr, *tb = nullptr;
  PyErr_Fetch(&type, &value, &tb);
  PyErr_NormalizeException(&type, &value, &tb);
  std::string msg = what;
  if (value) {
    if (PyObject* s = PyObject_Str(value)) {
      if (const char* c = PyUnicode_AsUTF8(s)) msg += std::string(": ") + c;
      Py_DECREF(s);
    }
  }
  Py_XDECREF(type);
  Py_XDECREF(value);
  Py_XDECREF(tb);
  PyErr_Clear();
  g_error = msg;
}

PyObject* capi_module() {
  PyObject* mod = PyImport_ImportModule("mythos_b200.capi");
  if (!mod) capture_python_error("cannot import mythos_b200.capi");
  return mod;
}

char* dup_cstr(const char* s) {
  const size_t n = std::strlen(s);
  char* out = static_cast<char*>(std::malloc(n + 1));
  if (out) std::memcpy(out, s, n + 1);
  return out;
}

}  // namespace

struct OilModel {
  PyObject* handle;  // mythos_b200.capi.Session
};

extern "C" {

const char* oil_last_error(void) { return g_error.c_str(); }

OilModel* oil_model_load_on(const char* path, const char* device) {
  g_error.clear();
  if (!path) {
    g_error = "oil_model_load: null path";
    return nullptr;
  }
  ensure_interpreter();
  Gil gil;
  PyObject* mod = capi_module();
  if (!mod) return nullptr;
  PyObject* h = PyObject_CallMethod(mod, "load", "ss", path, device ? device : "auto");
  Py_DECREF(mod);
  if (!h) {
    capture_python_error("oil_model_load failed");
    return nullptr;
  }
  OilModel* m = new OilModel{h};
  return m;
}

OilModel* oil_model_load(const char* path) { return oil_model_load_on(path, "auto"); }

void oil_model_free(OilModel* model) {
  if (!model) return;
  ensure_interpreter();
  {
    Gil gil;
    if (PyObject* r = PyObject_CallMethod(model->handle, "close", nullptr)) Py_DECREF(r);
    else PyErr_Clear();
    Py_DECREF(model->handle);
  }
  delete model;
}

char* oil_generate_sampled(OilModel* model, const char* prompt, int max_tokens, float temperature, int top_k,
                           float top_p, unsigned long long seed) {
  g_error.clear();
  if (!model || !prompt) {
    g_error = "oil_generate: null model or prompt";
    return nullptr;
  }
  ensure_interpreter();
  Gil gil;
  PyObject* r = PyObject_CallMethod(model->handle, "generate", "sididK", prompt, max_tokens,
                                    (double)temperature, top_k, (double)top_p, seed);
  if (!r) {
    capture_python_error("oil_generate failed");
    return nullptr;
  }
  char* out = nullptr;
  if (const char* c = PyUnicode_AsUTF8(r)) out = dup_cstr(c);
  else capture_python_error("oil_generate: result is not text");
  Py_DECREF(r);
  return out;
}

char* oil_generate(OilModel* model, const char* prompt, int max_tokens) {
  return oil_generate_sampled(model, prompt, max_tokens, 0.0f, 0, 1.0f, 0ull);
}

void oil_free_string(char* s) { std::free(s); }

int oil_generate_binding(const char* language, const char* output_dir) {
  (void)output_dir;
  g_error = std::string("binding generator for '") + (language ? language : "?") + "' is not implemented";
  return 0;
}

}  // extern "C"
