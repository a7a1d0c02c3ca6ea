// C interface of the engine (reflex_b200.h): marshals plain C values to the
// functions of reflex_b200.capi.bridge, run by an interpreter inside the
// calling process.  Status and error rules follow the reference's C interface
// (src/ffi.rs:20-32, include/reflex_engine.h:155-214): failures never cross as
// exceptions, the last error is thread-local and cleared by a success, result
// buffers belong to the library, free functions take NULL and zeroed structs.

#define PY_SSIZE_T_CLEAN
#include <Python.h>
#include <dlfcn.h>

#include <cstdlib>
#include <cstring>
#include <mutex>
#include <string>
#include <vector>

#include "reflex_b200.h"

#ifndef RFX_PYTHON_EXECUTABLE
#define RFX_PYTHON_EXECUTABLE ""
#endif

struct RfxModel {
    PyObject *model;  // reflex_b200.Model
};

namespace {

thread_local std::string tl_message;
thread_local RfxErrorCode tl_code = RFX_CODE_OK;
thread_local bool tl_failed = false;

void set_ok() {
    tl_failed = false;
    tl_code = RFX_CODE_OK;
    tl_message.clear();
}

void set_error(RfxErrorCode code, const std::string &message) {
    tl_failed = true;
    tl_code = code;
    tl_message = message;
}

std::once_flag g_once;
bool g_ready = false;
std::string g_start_error;
PyObject *g_bridge = nullptr;  // module reflex_b200.capi.bridge

// The folder that holds the package `reflex_b200`: this library lies somewhere
// below it, so walk up from the library's own path.
std::string package_root() {
    if (const char *env = std::getenv("REFLEX_B200_ROOT")) return env;
    Dl_info info;
    if (!dladdr(reinterpret_cast<void *>(&package_root), &info) || !info.dli_fname) return "";
    std::string path = info.dli_fname;
    for (int up = 0; up < 8; ++up) {
        size_t cut = path.find_last_of('/');
        if (cut == std::string::npos || cut == 0) break;
        path.resize(cut);
        std::string probe = path + "/reflex_b200/__init__.py";
        if (FILE *f = std::fopen(probe.c_str(), "r")) {
            std::fclose(f);
            return path;
        }
    }
    return "";
}

void start_interpreter() {
    bool ours = false;
    PyGILState_STATE gil{};
    if (!Py_IsInitialized()) {
        PyConfig config;
        PyConfig_InitPythonConfig(&config);
        // The interpreter this library was built with; its environment (a
        // virtual environment's packages) is found from the executable's place.
        const char *exe = std::getenv("REFLEX_B200_PYTHON");
        if (!exe || !*exe) exe = RFX_PYTHON_EXECUTABLE;
        if (exe && *exe) {
            PyStatus st = PyConfig_SetBytesString(&config, &config.executable, exe);
            if (!PyStatus_Exception(st)) st = PyConfig_SetBytesString(&config, &config.program_name, exe);
            if (PyStatus_Exception(st)) {
                PyConfig_Clear(&config);
                g_start_error = "could not configure the interpreter's executable";
                return;
            }
        }
        config.install_signal_handlers = 0;
        config.parse_argv = 0;
        PyStatus st = Py_InitializeFromConfig(&config);
        PyConfig_Clear(&config);
        if (PyStatus_Exception(st)) {
            g_start_error = std::string("the interpreter did not start: ") + (st.err_msg ? st.err_msg : "?");
            return;
        }
        ours = true;
    } else {
        gil = PyGILState_Ensure();
    }

    std::string root = package_root();
    if (!root.empty()) {
        PyObject *sys_path = PySys_GetObject("path");  // borrowed
        PyObject *entry = PyUnicode_FromString(root.c_str());
        if (sys_path && entry && !PySequence_Contains(sys_path, entry)) PyList_Insert(sys_path, 0, entry);
        Py_XDECREF(entry);
    }
    g_bridge = PyImport_ImportModule("reflex_b200.capi.bridge");
    if (!g_bridge) {
        PyObject *type, *value, *tb;
        PyErr_Fetch(&type, &value, &tb);
        PyObject *text = value ? PyObject_Str(value) : nullptr;
        const char *msg = text ? PyUnicode_AsUTF8(text) : nullptr;
        g_start_error = std::string("cannot import reflex_b200.capi.bridge: ") + (msg ? msg : "?");
        PyErr_Clear();
        Py_XDECREF(text);
        Py_XDECREF(type);
        Py_XDECREF(value);
        Py_XDECREF(tb);
    } else {
        g_ready = true;
    }
    if (ours)
        PyEval_SaveThread();  // later calls take the interpreter lock themselves
    else
        PyGILState_Release(gil);
}

bool ensure_started() {
    std::call_once(g_once, start_interpreter);
    if (!g_ready) set_error(RFX_CODE_OTHER, g_start_error.empty() ? "the engine did not start" : g_start_error);
    return g_ready;
}

// Holds the interpreter lock for a scope.
struct Gil {
    PyGILState_STATE state;
    Gil() : state(PyGILState_Ensure()) {}
    ~Gil() { PyGILState_Release(state); }
};

// Records the pending Python exception as the thread's last error.
void take_python_error() {
    PyObject *type, *value, *tb;
    PyErr_Fetch(&type, &value, &tb);
    PyErr_NormalizeException(&type, &value, &tb);
    long code = RFX_CODE_OTHER;
    std::string message = "unknown failure";
    if (value && g_bridge) {
        PyObject *info = PyObject_CallMethod(g_bridge, "describe_error", "O", value);
        if (info && PyTuple_Check(info) && PyTuple_GET_SIZE(info) == 2) {
            code = PyLong_AsLong(PyTuple_GET_ITEM(info, 0));
            if (const char *m = PyUnicode_AsUTF8(PyTuple_GET_ITEM(info, 1))) message = m;
        }
        Py_XDECREF(info);
        PyErr_Clear();
    }
    if (code < 0 || code > 14) code = RFX_CODE_OTHER;
    set_error(static_cast<RfxErrorCode>(code), message);
    Py_XDECREF(type);
    Py_XDECREF(value);
    Py_XDECREF(tb);
}

PyObject *id_list(const uint32_t *ids, size_t n) {
    PyObject *list = PyList_New(static_cast<Py_ssize_t>(n));
    if (!list) return nullptr;
    for (size_t i = 0; i < n; ++i) {
        PyObject *v = PyLong_FromUnsignedLong(ids[i]);
        if (!v) {
            Py_DECREF(list);
            return nullptr;
        }
        PyList_SET_ITEM(list, static_cast<Py_ssize_t>(i), v);
    }
    return list;
}

PyObject *id_lists(const uint32_t *const *rows, const size_t *lens, size_t n) {
    PyObject *outer = PyList_New(static_cast<Py_ssize_t>(n));
    if (!outer) return nullptr;
    for (size_t i = 0; i < n; ++i) {
        PyObject *inner = id_list(rows[i], lens[i]);
        if (!inner) {
            Py_DECREF(outer);
            return nullptr;
        }
        PyList_SET_ITEM(outer, static_cast<Py_ssize_t>(i), inner);
    }
    return outer;
}

bool check_rows(const uint32_t *const *rows, const size_t *lens, size_t n, const char *what) {
    if (n == 0) return true;
    if (!rows || !lens) {
        set_error(RFX_CODE_INVALID_INPUT, std::string(what) + " is NULL");
        return false;
    }
    for (size_t i = 0; i < n; ++i)
        if (lens[i] > 0 && !rows[i]) {
            set_error(RFX_CODE_INVALID_INPUT, std::string(what) + " holds a NULL row");
            return false;
        }
    return true;
}

RfxModel *wrap_model(PyObject *model) {
    if (!model) {
        take_python_error();
        return nullptr;
    }
    RfxModel *handle = static_cast<RfxModel *>(std::calloc(1, sizeof(RfxModel)));
    if (!handle) {
        Py_DECREF(model);
        set_error(RFX_CODE_OUT_OF_MEMORY, "out of host memory");
        return nullptr;
    }
    handle->model = model;
    set_ok();
    return handle;
}

}  // namespace

extern "C" {

const char *rfx_last_error(void) { return tl_failed ? tl_message.c_str() : nullptr; }

RfxErrorCode rfx_last_error_code(void) { return tl_failed ? tl_code : RFX_CODE_OK; }

RfxModel *rfx_load(const char *model_dir, const char *weights, size_t max_tokens, size_t max_batch) {
    if (!model_dir) {
        set_error(RFX_CODE_INVALID_INPUT, "model_dir is NULL");
        return nullptr;
    }
    if (!ensure_started()) return nullptr;
    Gil gil;
    return wrap_model(PyObject_CallMethod(g_bridge, "load", "ssnn", model_dir, weights ? weights : "bf16",
                                          static_cast<Py_ssize_t>(max_tokens),
                                          static_cast<Py_ssize_t>(max_batch)));
}

RfxModel *rfx_load_random(const char *config_json, uint64_t seed, const char *out_dir, const char *weights,
                          size_t max_tokens, size_t max_batch) {
    if (!config_json || !out_dir) {
        set_error(RFX_CODE_INVALID_INPUT, config_json ? "out_dir is NULL" : "config_json is NULL");
        return nullptr;
    }
    if (!ensure_started()) return nullptr;
    Gil gil;
    return wrap_model(PyObject_CallMethod(g_bridge, "load_random", "sKssnn", config_json,
                                          static_cast<unsigned long long>(seed), out_dir,
                                          weights ? weights : "bf16", static_cast<Py_ssize_t>(max_tokens),
                                          static_cast<Py_ssize_t>(max_batch)));
}

void rfx_free(RfxModel *model) {
    if (!model) return;
    if (model->model && g_ready) {
        Gil gil;
        Py_CLEAR(model->model);
    }
    std::free(model);
}

int rfx_generate(RfxModel *model, const uint32_t *const *prompts, const size_t *prompt_lens,
                 size_t num_prompts, size_t max_new_tokens, const RfxSampling *sampling,
                 RfxGenerateResult *out) {
    if (out) std::memset(out, 0, sizeof(*out));
    if (!model || !model->model || !out) {
        set_error(RFX_CODE_INVALID_INPUT, !out ? "out is NULL" : "model is NULL");
        return -1;
    }
    if (!check_rows(prompts, prompt_lens, num_prompts, "prompts")) return -1;
    if (sampling && sampling->num_stop_token_ids > 0 && !sampling->stop_token_ids) {
        set_error(RFX_CODE_INVALID_INPUT, "stop_token_ids is NULL");
        return -1;
    }
    if (!ensure_started()) return -1;
    Gil gil;
    PyObject *plist = id_lists(prompts, prompt_lens, num_prompts);
    PyObject *stops = sampling ? id_list(sampling->stop_token_ids, sampling->num_stop_token_ids) : PyList_New(0);
    PyObject *result = nullptr;
    if (plist && stops)
        result = PyObject_CallMethod(g_bridge, "generate", "OOndidLO", model->model, plist,
                                     static_cast<Py_ssize_t>(max_new_tokens),
                                     sampling ? static_cast<double>(sampling->temperature) : 0.0,
                                     sampling ? static_cast<int>(sampling->top_k) : 0,
                                     sampling ? static_cast<double>(sampling->top_p) : 0.0,
                                     sampling ? static_cast<long long>(sampling->seed) : -1LL, stops);
    Py_XDECREF(plist);
    Py_XDECREF(stops);
    if (!result) {
        take_python_error();
        return -1;
    }
    size_t n = static_cast<size_t>(PyList_Size(result));
    RfxSequence *seqs = static_cast<RfxSequence *>(std::calloc(n ? n : 1, sizeof(RfxSequence)));
    bool ok = seqs != nullptr;
    for (size_t i = 0; ok && i < n; ++i) {
        PyObject *row = PyList_GetItem(result, static_cast<Py_ssize_t>(i));  // borrowed
        size_t len = static_cast<size_t>(PyList_Size(row));
        seqs[i].token_ids = static_cast<uint32_t *>(std::calloc(len ? len : 1, sizeof(uint32_t)));
        if (!seqs[i].token_ids) {
            ok = false;
            break;
        }
        seqs[i].num_tokens = len;
        for (size_t j = 0; j < len; ++j)
            seqs[i].token_ids[j] =
                static_cast<uint32_t>(PyLong_AsUnsignedLong(PyList_GetItem(row, static_cast<Py_ssize_t>(j))));
    }
    Py_DECREF(result);
    out->sequences = seqs;
    out->num_sequences = seqs ? n : 0;
    if (!ok) {
        rfx_free_generate_result(out);
        set_error(RFX_CODE_OUT_OF_MEMORY, "out of host memory");
        return -1;
    }
    set_ok();
    return 0;
}

void rfx_free_generate_result(RfxGenerateResult *result) {
    if (!result) return;
    if (result->sequences) {
        for (size_t i = 0; i < result->num_sequences; ++i) std::free(result->sequences[i].token_ids);
        std::free(result->sequences);
    }
    result->sequences = nullptr;
    result->num_sequences = 0;
}

int rfx_score(RfxModel *model, const uint32_t *prompt, size_t prompt_len, const uint32_t *const *candidates,
              const size_t *candidate_lens, size_t num_candidates, float temperature, RfxScoreResult *out) {
    if (out) std::memset(out, 0, sizeof(*out));
    if (!model || !model->model || !out) {
        set_error(RFX_CODE_INVALID_INPUT, !out ? "out is NULL" : "model is NULL");
        return -1;
    }
    if (prompt_len > 0 && !prompt) {
        set_error(RFX_CODE_INVALID_INPUT, "prompt is NULL");
        return -1;
    }
    if (!check_rows(candidates, candidate_lens, num_candidates, "candidates")) return -1;
    if (!ensure_started()) return -1;
    Gil gil;
    PyObject *p = id_list(prompt, prompt_len);
    PyObject *c = id_lists(candidates, candidate_lens, num_candidates);
    PyObject *result = nullptr;
    if (p && c)
        result = PyObject_CallMethod(g_bridge, "score", "OOOd", model->model, p, c, static_cast<double>(temperature));
    Py_XDECREF(p);
    Py_XDECREF(c);
    if (!result) {
        take_python_error();
        return -1;
    }
    PyObject *scores = PyTuple_GetItem(result, 0), *probs = PyTuple_GetItem(result, 1);  // borrowed
    size_t n = static_cast<size_t>(PyList_Size(scores));
    RfxCandidateScore *rows = static_cast<RfxCandidateScore *>(std::calloc(n ? n : 1, sizeof(RfxCandidateScore)));
    if (!rows) {
        Py_DECREF(result);
        set_error(RFX_CODE_OUT_OF_MEMORY, "out of host memory");
        return -1;
    }
    for (size_t i = 0; i < n; ++i) {
        rows[i].score = static_cast<float>(PyFloat_AsDouble(PyList_GetItem(scores, static_cast<Py_ssize_t>(i))));
        rows[i].probability = static_cast<float>(PyFloat_AsDouble(PyList_GetItem(probs, static_cast<Py_ssize_t>(i))));
    }
    out->candidates = rows;
    out->num_candidates = n;
    out->best_idx = static_cast<size_t>(PyLong_AsLong(PyTuple_GetItem(result, 2)));
    out->entropy = static_cast<float>(PyFloat_AsDouble(PyTuple_GetItem(result, 3)));
    Py_DECREF(result);
    set_ok();
    return 0;
}

void rfx_free_score_result(RfxScoreResult *result) {
    if (!result) return;
    std::free(result->candidates);
    result->candidates = nullptr;
    result->num_candidates = 0;
}

int rfx_open_sequence(RfxModel *model, int64_t *sequence) {
    if (!model || !model->model || !sequence) {
        set_error(RFX_CODE_INVALID_INPUT, !sequence ? "sequence is NULL" : "model is NULL");
        return -1;
    }
    if (!ensure_started()) return -1;
    Gil gil;
    PyObject *r = PyObject_CallMethod(g_bridge, "open_sequence", "O", model->model);
    if (!r) {
        take_python_error();
        return -1;
    }
    *sequence = static_cast<int64_t>(PyLong_AsLongLong(r));
    Py_DECREF(r);
    set_ok();
    return 0;
}

int rfx_close_sequence(RfxModel *model, int64_t sequence) {
    if (!model || !model->model) {
        set_error(RFX_CODE_INVALID_INPUT, "model is NULL");
        return -1;
    }
    if (!ensure_started()) return -1;
    Gil gil;
    PyObject *r = PyObject_CallMethod(g_bridge, "close_sequence", "OL", model->model, static_cast<long long>(sequence));
    if (!r) {
        take_python_error();
        return -1;
    }
    Py_DECREF(r);
    set_ok();
    return 0;
}

int rfx_step(RfxModel *model, const RfxStepEntry *entries, size_t num_entries, RfxStepResult *out) {
    if (out) std::memset(out, 0, sizeof(*out));
    if (!model || !model->model || !out || (num_entries > 0 && !entries)) {
        set_error(RFX_CODE_INVALID_INPUT, !out ? "out is NULL" : (!model || !model->model) ? "model is NULL" : "entries is NULL");
        return -1;
    }
    for (size_t i = 0; i < num_entries; ++i)
        if ((entries[i].num_tokens > 0 && !entries[i].tokens) || (entries[i].num_want > 0 && !entries[i].want)) {
            set_error(RFX_CODE_INVALID_INPUT, "an entry holds a NULL array");
            return -1;
        }
    if (!ensure_started()) return -1;
    Gil gil;
    PyObject *list = PyList_New(static_cast<Py_ssize_t>(num_entries));
    bool ok = list != nullptr;
    for (size_t i = 0; ok && i < num_entries; ++i) {
        PyObject *t = id_list(entries[i].tokens, entries[i].num_tokens);
        PyObject *w = id_list(entries[i].want, entries[i].num_want);
        PyObject *tup = (t && w) ? Py_BuildValue("(LOO)", static_cast<long long>(entries[i].sequence), t, w) : nullptr;
        Py_XDECREF(t);
        Py_XDECREF(w);
        if (!tup) {
            ok = false;
            break;
        }
        PyList_SET_ITEM(list, static_cast<Py_ssize_t>(i), tup);
    }
    PyObject *result = ok ? PyObject_CallMethod(g_bridge, "step", "OO", model->model, list) : nullptr;
    Py_XDECREF(list);
    if (!result) {
        take_python_error();
        return -1;
    }
    size_t rows = static_cast<size_t>(PyLong_AsLong(PyTuple_GetItem(result, 0)));
    size_t vocab = static_cast<size_t>(PyLong_AsLong(PyTuple_GetItem(result, 1)));
    PyObject *bytes = PyTuple_GetItem(result, 2);  // borrowed
    if (rows > 0 && PyBytes_Check(bytes)) {
        size_t size = static_cast<size_t>(PyBytes_GET_SIZE(bytes));
        out->logits = static_cast<float *>(std::malloc(size ? size : 1));
        if (!out->logits) {
            Py_DECREF(result);
            set_error(RFX_CODE_OUT_OF_MEMORY, "out of host memory");
            return -1;
        }
        std::memcpy(out->logits, PyBytes_AS_STRING(bytes), size);
    }
    out->rows = rows;
    out->vocab = vocab;
    Py_DECREF(result);
    set_ok();
    return 0;
}

void rfx_free_step_result(RfxStepResult *result) {
    if (!result) return;
    std::free(result->logits);
    result->logits = nullptr;
    result->rows = 0;
}

}  // extern "C"
