// libqw_engine.so: the C ABI of include/qw/capi.h over the Python engine.
//
// PyTorch is the framework layer of this engine, so the shim forwards every call to one method of a
// Python object (qwb200.capi_impl.CApi) through the CPython API: when the host is a Python process
// (the qwserve server loads this library with ctypes) the interpreter is already there; a C host gets
// an embedded interpreter on the first qw_open.  Pointers cross the boundary as integers and the
// Python side reads / writes the caller's buffers with ctypes, so no data is copied here.  Python
// exceptions become -1 with the message kept for qw_error (the role of the reference's `guarded()`,
// src/capi/capi.cpp:21-30).
#include <Python.h>

#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <string>

#include "qw/capi.h"

struct qw_handle {
    PyObject *obj = nullptr;
    std::string error;
    std::mutex fail_mu;
};

namespace {

bool g_we_initialized = false;

struct Gil {
    PyGILState_STATE st;
    Gil() : st(PyGILState_Ensure()) {}
    ~Gil() { PyGILState_Release(st); }
};

void ensure_python() {
    if (!Py_IsInitialized()) {
        Py_InitializeEx(0);
        g_we_initialized = true;
        PyEval_SaveThread();          // release the GIL: every call takes it again through Gil
    }
}

std::string take_error() {
    PyObject *t = nullptr, *v = nullptr, *tb = nullptr;
    PyErr_Fetch(&t, &v, &tb);
    PyErr_NormalizeException(&t, &v, &tb);
    std::string msg = "python error";
    if (v) {
        if (PyObject *s = PyObject_Str(v)) {
            if (const char *c = PyUnicode_AsUTF8(s)) msg = c;
            Py_DECREF(s);
        }
    }
    Py_XDECREF(t); Py_XDECREF(v); Py_XDECREF(tb);
    return msg;
}

// Calls h->obj.<name>(*args built from fmt) and returns the result as long long; -1 on a Python exception.
long long call(qw_handle *h, const char *name, const char *fmt, ...) {
    if (!h || !h->obj) return -1;
    Gil gil;
    va_list ap;
    va_start(ap, fmt);
    PyObject *args = Py_VaBuildValue(fmt, ap);
    va_end(ap);
    PyObject *res = nullptr;
    if (args) {
        if (PyObject *m = PyObject_GetAttrString(h->obj, name)) {
            res = PyObject_CallObject(m, args);
            Py_DECREF(m);
        }
        Py_DECREF(args);
    }
    if (!res) {
        h->error = take_error();
        return -1;
    }
    h->error.clear();
    long long v = 0;
    if (res != Py_None) {
        v = PyLong_AsLongLong(res);
        if (PyErr_Occurred()) { h->error = take_error(); v = -1; }
    }
    Py_DECREF(res);
    return v;
}
#define PTR(p) ((long long)(intptr_t)(p))

}  // namespace

extern "C" {

qw_handle *qw_open(const char *options_json, char *err, int errlen) {
    ensure_python();
    Gil gil;
    auto fail = [&](const std::string &m) -> qw_handle * {
        if (err && errlen > 0) std::snprintf(err, size_t(errlen), "%s", m.c_str());
        return nullptr;
    };
    PyObject *mod = PyImport_ImportModule("qwb200.capi_impl");
    if (!mod) return fail(take_error());
    PyObject *obj = PyObject_CallMethod(mod, "open", "s", options_json ? options_json : "{}");
    Py_DECREF(mod);
    if (!obj) return fail(take_error());
    auto *h = new qw_handle();
    h->obj = obj;
    return h;
}

void qw_close(qw_handle *h) {
    if (!h) return;
    call(h, "close", "()");
    {
        Gil gil;
        Py_XDECREF(h->obj);
    }
    delete h;
}

int qw_persist(qw_handle *h) { return (int)call(h, "persist", "()"); }
const char *qw_error(qw_handle *h) { return h ? h->error.c_str() : "null handle"; }

int qw_engine_failure(qw_handle *h, char *buf, int buflen) {
    if (!h) return 0;
    std::lock_guard<std::mutex> lk(h->fail_mu);
    Gil gil;
    PyObject *res = PyObject_CallMethod(h->obj, "failure", "()");
    if (!res) { PyErr_Clear(); return 0; }
    int n = 0;
    if (const char *c = PyUnicode_Check(res) ? PyUnicode_AsUTF8(res) : nullptr) {
        n = (int)std::strlen(c);
        if (buf && buflen > 0) std::snprintf(buf, size_t(buflen), "%s", c);
    }
    Py_DECREF(res);
    return n;
}

int qw_set_boundary_token(qw_handle *h, int32_t id) { return (int)call(h, "set_boundary_token", "(i)", (int)id); }
int qw_get_cache_stats(qw_handle *h, qw_cache_stats *out) { return (int)call(h, "get_cache_stats", "(L)", PTR(out)); }
int qw_get_slot_timing(qw_handle *h, int slot, qw_slot_timing *out) { return (int)call(h, "get_slot_timing", "(iL)", slot, PTR(out)); }
int qw_num_slots(qw_handle *h) { return (int)call(h, "num_slots", "()"); }
int64_t qw_slot_capacity(qw_handle *h, int slot) { return call(h, "slot_capacity", "(i)", slot); }

int qw_acquire(qw_handle *h, const int32_t *tokens, int64_t n, int64_t max_new) {
    return (int)call(h, "acquire", "(LLLLi)", PTR(tokens), (long long)n, (long long)max_new, 0LL, 0);
}
int qw_acquire_media(qw_handle *h, const int32_t *tokens, int64_t n, int64_t max_new, const qw_media *media, int n_media) {
    return (int)call(h, "acquire", "(LLLLi)", PTR(tokens), (long long)n, (long long)max_new, PTR(media), n_media);
}
int qw_release(qw_handle *h, int slot) { return (int)call(h, "release", "(i)", slot); }
int64_t qw_set_prompt(qw_handle *h, int slot, const int32_t *tokens, int64_t n) {
    return call(h, "set_prompt", "(iLLLi)", slot, PTR(tokens), (long long)n, 0LL, 0);
}
int64_t qw_set_prompt_media(qw_handle *h, int slot, const int32_t *tokens, int64_t n, const qw_media *media, int n_media) {
    return call(h, "set_prompt", "(iLLLi)", slot, PTR(tokens), (long long)n, PTR(media), n_media);
}
int qw_has_vision(qw_handle *h) { return (int)call(h, "has_vision", "()"); }
int64_t qw_begin_prompt(qw_handle *h, int slot, const int32_t *tokens, int64_t n, const qw_media *media, int n_media) {
    return call(h, "begin_prompt", "(iLLLi)", slot, PTR(tokens), (long long)n, PTR(media), n_media);
}
int qw_prefill_some(qw_handle *h, int slot, int64_t max_tokens) { return (int)call(h, "prefill_some", "(iL)", slot, (long long)max_tokens); }
int qw_prefetch(qw_handle *h, int slot, const int32_t *tokens, int64_t n, const qw_media *media, int n_media) {
    return (int)call(h, "prefetch", "(iLLLi)", slot, PTR(tokens), (long long)n, PTR(media), n_media);
}
int qw_prefill_batch(qw_handle *h, int n, const int32_t *slots, const int64_t *max_tokens, int32_t *done) {
    return (int)call(h, "prefill_batch", "(iLLL)", n, PTR(slots), PTR(max_tokens), PTR(done));
}
int32_t qw_sample_prompt(qw_handle *h, int slot, const qw_sampling *p, float *lp) {
    return (int32_t)call(h, "sample_prompt", "(iLL)", slot, PTR(p), PTR(lp));
}
int qw_decode(qw_handle *h, int n, const int32_t *slots, const int32_t *tokens) {
    return (int)call(h, "decode", "(iLL)", n, PTR(slots), PTR(tokens));
}
int32_t qw_sample_row(qw_handle *h, int row, const qw_sampling *p, float *lp) {
    return (int32_t)call(h, "sample_row", "(iLL)", row, PTR(p), PTR(lp));
}
int qw_has_mtp(qw_handle *h) { return (int)call(h, "has_mtp", "()"); }
int qw_set_stop_tokens(qw_handle *h, int slot, const int32_t *ids, int n) { return (int)call(h, "set_stop_tokens", "(iLi)", slot, PTR(ids), n); }
int qw_generate(qw_handle *h, int n, const qw_step_req *reqs, int k, int32_t *tokens, float *logprobs, int32_t *counts,
                int32_t *first_rows, int32_t *stopped) {
    return (int)call(h, "generate", "(iLiLLLLL)", n, PTR(reqs), k, PTR(tokens), PTR(logprobs), PTR(counts), PTR(first_rows), PTR(stopped));
}
int qw_top_logprobs(qw_handle *h, int row, int k, int32_t *ids, float *lps) {
    return (int)call(h, "top_logprobs", "(iiLL)", row, k, PTR(ids), PTR(lps));
}
int qw_top_logprobs_prompt(qw_handle *h, int slot, int k, int32_t *ids, float *lps) {
    return (int)call(h, "top_logprobs_prompt", "(iiLL)", slot, k, PTR(ids), PTR(lps));
}

}  // extern "C"
