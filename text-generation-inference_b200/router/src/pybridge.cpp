#include "pybridge.hpp"

#include <Python.h>

#include <mutex>
#include <stdexcept>

namespace bridge {

namespace {
PyObject* g_module = nullptr;
PyThreadState* g_main = nullptr;
std::once_flag g_once;

std::string py_error() {
  PyObject *type, *value, *tb;
  PyErr_Fetch(&type, &value, &tb);
  PyErr_NormalizeException(&type, &value, &tb);
  std::string msg = "python error";
  if (value) {
    PyObject* s = PyObject_Str(value);
    if (s) {
      const char* c = PyUnicode_AsUTF8(s);
      if (c) msg = c;
      Py_DECREF(s);
    }
  }
  Py_XDECREF(type);
  Py_XDECREF(value);
  Py_XDECREF(tb);
  return msg;
}
}  // namespace

void init(const std::string& repo_root) {
  std::call_once(g_once, [&] {
    Py_InitializeEx(0);
    PyObject* sys_path = PySys_GetObject("path");
    PyObject* p = PyUnicode_FromString(repo_root.c_str());
    PyList_Insert(sys_path, 0, p);
    Py_DECREF(p);
    // a virtualenv's site-packages is not on the default path of an embedded interpreter
    PyRun_SimpleString(
        "import os, site, sys\n"
        "venv = os.environ.get('VIRTUAL_ENV')\n"
        "cands = [os.path.join(venv, 'lib', 'python%d.%d' % sys.version_info[:2], 'site-packages')] if venv else []\n"
        "cands += [p for p in os.environ.get('TGI_B200_SITE_PACKAGES', '').split(':') if p]\n"
        "for c in cands:\n"
        "    if os.path.isdir(c): site.addsitedir(c)\n");
    g_module = PyImport_ImportModule("tgi_b200.router.pybridge");
    if (!g_module) {
      std::string e = py_error();
      throw std::runtime_error("cannot import tgi_b200.router.pybridge: " + e);
    }
    g_main = PyEval_SaveThread();   // release the GIL; callers take it per call
  });
}

void shutdown() {
  if (g_main) {
    PyEval_RestoreThread(g_main);
    Py_XDECREF(g_module);
    g_module = nullptr;
    Py_FinalizeEx();
    g_main = nullptr;
  }
}

json::Value call(const char* fn, const json::Value& arg) {
  if (!g_module) throw std::runtime_error("python bridge is not initialised");
  PyGILState_STATE st = PyGILState_Ensure();
  std::string out, err;
  PyObject* f = PyObject_GetAttrString(g_module, fn);
  if (!f) {
    err = py_error();
  } else {
    const std::string payload = arg.dump();
    PyObject* a = PyUnicode_FromStringAndSize(payload.data(), static_cast<Py_ssize_t>(payload.size()));
    PyObject* r = a ? PyObject_CallFunctionObjArgs(f, a, nullptr) : nullptr;
    if (!r) {
      err = py_error();
    } else {
      Py_ssize_t n = 0;
      const char* c = PyUnicode_AsUTF8AndSize(r, &n);
      if (c) out.assign(c, static_cast<size_t>(n));
      else err = py_error();
      Py_DECREF(r);
    }
    Py_XDECREF(a);
    Py_DECREF(f);
  }
  PyGILState_Release(st);
  if (!err.empty()) throw std::runtime_error(std::string(fn) + ": " + err);
  return json::Value::parse(out);
}

}  // namespace bridge
