// C API over the Python inference engine (see tfb_capi.h).
#include "tfb_capi.h"

#include <Python.h>
#include <stdlib.h>
#include <string.h>

#include <mutex>
#include <string>

#define TFB_EXPORT extern "C" __attribute__((visibility("default")))

namespace {

thread_local std::string g_err;
std::once_flag g_init;
bool g_we_started = false;

void ensure_python() {
  std::call_once(g_init, [] {
    if (!Py_IsInitialized()) {
      Py_InitializeEx(0);
      g_we_started = true;
      const char* extra = getenv("TFB_PYTHONPATH");
      if (extra && *extra) {
        PyObject* sys_path = PySys_GetObject("path");   // borrowed
        PyObject* p = PyUnicode_FromString(extra);
        if (sys_path && p) PyList_Insert(sys_path, 0, p);
        Py_XDECREF(p);
      }
      PyEval_SaveThread();   // release the lock; every call takes it with PyGILState_Ensure
    }
  });
}

void capture_error(const char* what) {
  g_err = what;
  if (PyErr_Occurred()) {
    PyObject *t = nullptr, *v = nullptr, *tb = nullptr;
    PyErr_Fetch(&t, &v, &tb);
    PyErr_NormalizeException(&t, &v, &tb);
    if (v) {
      PyObject* s = PyObject_Str(v);
      if (s) {
        const char* c = PyUnicode_AsUTF8(s);
        if (c) g_err += std::string(": ") + c;
        Py_DECREF(s);
      }
    }
    Py_XDECREF(t);
    Py_XDECREF(v);
    Py_XDECREF(tb);
    PyErr_Clear();
  }
}

}  // namespace

struct quant_model {
  PyObject* handle;   // transformers_fusion_b200.capi.Handle
};

TFB_EXPORT const char* quant_last_error(void) { return g_err.c_str(); }

TFB_EXPORT quant_model* quant_model_load(const char* path) {
  g_err.clear();
  if (!path) { g_err = "null path"; return nullptr; }
  ensure_python();
  PyGILState_STATE gs = PyGILState_Ensure();
  quant_model* out = nullptr;
  PyObject* mod = PyImport_ImportModule("transformers_fusion_b200.capi");
  if (!mod) capture_error("cannot import transformers_fusion_b200.capi");
  else {
    PyObject* h = PyObject_CallMethod(mod, "load", "s", path);
    if (!h) capture_error("load failed");
    else {
      out = new quant_model{h};
    }
    Py_DECREF(mod);
  }
  PyGILState_Release(gs);
  return out;
}

TFB_EXPORT void quant_model_free(quant_model* m) {
  if (!m) return;
  PyGILState_STATE gs = PyGILState_Ensure();
  Py_XDECREF(m->handle);
  PyGILState_Release(gs);
  delete m;
}

TFB_EXPORT char* quant_generate(quant_model* m, const char* prompt, int max_tokens, float temperature, int top_k, float top_p) {
  g_err.clear();
  if (!m || !prompt) { g_err = "null argument"; return nullptr; }
  PyGILState_STATE gs = PyGILState_Ensure();
  char* out = nullptr;
  PyObject* r = PyObject_CallMethod(m->handle, "generate", "sifif", prompt, max_tokens, double(temperature), top_k, double(top_p));
  if (!r) capture_error("generate failed");
  else {
    Py_ssize_t n = 0;
    const char* c = PyUnicode_AsUTF8AndSize(r, &n);
    if (!c) capture_error("result is not text");
    else {
      out = static_cast<char*>(malloc(size_t(n) + 1));
      if (out) { memcpy(out, c, size_t(n)); out[n] = 0; } else g_err = "out of memory";
    }
    Py_DECREF(r);
  }
  PyGILState_Release(gs);
  return out;
}

TFB_EXPORT void quant_free_string(char* s) { free(s); }
