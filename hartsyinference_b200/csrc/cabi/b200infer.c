/* Implementation of the C ABI: hosts (or joins) a CPython interpreter and forwards every call to
 * hartsyinference_b200.cabi, which owns the engine objects. See b200infer.h. */
#define PY_SSIZE_T_CLEAN
#include <Python.h>
#include <stdlib.h>
#include <string.h>

#include "b200infer.h"

struct b200_engine { long long handle; };

static __thread char g_err[2048];
static int g_we_initialised = 0;
static PyObject* g_mod = NULL;

static void set_err(const char* msg) {
  strncpy(g_err, msg ? msg : "unknown error", sizeof(g_err) - 1);
  g_err[sizeof(g_err) - 1] = 0;
}

static int ensure_python(PyGILState_STATE* st) {
  if (!Py_IsInitialized()) {
    Py_InitializeEx(0);
    g_we_initialised = 1;
    /* release the GIL acquired by initialisation so that PyGILState_Ensure works from any thread */
    PyEval_SaveThread();
  }
  *st = PyGILState_Ensure();
  if (g_mod == NULL) {
    g_mod = PyImport_ImportModule("hartsyinference_b200.cabi");
    if (g_mod == NULL) {
      PyErr_Print();
      set_err("cannot import hartsyinference_b200.cabi (is the package on PYTHONPATH?)");
      PyGILState_Release(*st);
      return 1;
    }
  }
  return 0;
}

/* Calls module function `name`; the Python side returns (code, message, payload). */
static int call(const char* name, PyObject* args, PyObject** payload) {
  PyObject* fn = PyObject_GetAttrString(g_mod, name);
  if (!fn) { PyErr_Clear(); set_err("missing cabi function"); Py_XDECREF(args); return 1; }
  PyObject* res = PyObject_CallObject(fn, args);
  Py_DECREF(fn);
  Py_XDECREF(args);
  if (!res) {
    PyObject *t, *v, *tb;
    PyErr_Fetch(&t, &v, &tb);
    PyObject* s = v ? PyObject_Str(v) : NULL;
    set_err(s ? PyUnicode_AsUTF8(s) : "python exception");
    Py_XDECREF(s); Py_XDECREF(t); Py_XDECREF(v); Py_XDECREF(tb);
    return 1;
  }
  int code = (int)PyLong_AsLong(PyTuple_GetItem(res, 0));
  if (code != 0) {
    const char* m = PyUnicode_AsUTF8(PyTuple_GetItem(res, 1));
    set_err(m);
  }
  if (payload) { *payload = PyTuple_GetItem(res, 2); Py_INCREF(*payload); }
  Py_DECREF(res);
  return code;
}

static char* dup_str(PyObject* o) {
  Py_ssize_t n = 0;
  const char* s = PyUnicode_AsUTF8AndSize(o, &n);
  char* out = (char*)malloc((size_t)n + 1);
  if (out) { memcpy(out, s ? s : "", (size_t)n); out[n] = 0; }
  return out;
}

#define ENTER() PyGILState_STATE gst; if (ensure_python(&gst)) return 7
#define LEAVE(code) do { PyGILState_Release(gst); return (code); } while (0)

int b200_engine_create(const char* selector, const char* options_json, b200_engine** out) {
  ENTER();
  PyObject* p = NULL;
  int rc = call("engine_create", Py_BuildValue("(ss)", selector ? selector : "auto", options_json ? options_json : "{}"), &p);
  if (rc == 0) {
    b200_engine* e = (b200_engine*)malloc(sizeof(*e));
    e->handle = PyLong_AsLongLong(p);
    *out = e;
  }
  Py_XDECREF(p);
  LEAVE(rc);
}

void b200_engine_destroy(b200_engine* e) {
  if (!e) return;
  PyGILState_STATE gst;
  if (ensure_python(&gst)) return;
  call("engine_destroy", Py_BuildValue("(L)", e->handle), NULL);
  PyGILState_Release(gst);
  free(e);
}

int b200_engine_set_backend(b200_engine* e, const char* selector) {
  ENTER();
  int rc = call("engine_set_backend", Py_BuildValue("(Ls)", e->handle, selector), NULL);
  LEAVE(rc);
}

int b200_engine_describe(b200_engine* e, char** json_out) {
  ENTER();
  PyObject* p = NULL;
  int rc = call("engine_describe", Py_BuildValue("(L)", e->handle), &p);
  if (rc == 0 && json_out) *json_out = dup_str(p);
  Py_XDECREF(p);
  LEAVE(rc);
}

int b200_engine_is_supported(b200_engine* e, const char* modality) {
  PyGILState_STATE gst;
  if (ensure_python(&gst)) return 0;
  PyObject* p = NULL;
  int rc = call("engine_is_supported", Py_BuildValue("(Ls)", e->handle, modality), &p);
  int yes = rc == 0 && p && PyObject_IsTrue(p);
  Py_XDECREF(p);
  PyGILState_Release(gst);
  return yes;
}

int b200_free_memory(b200_engine* e) {
  ENTER();
  int rc = call("free_memory", Py_BuildValue("(L)", e->handle), NULL);
  LEAVE(rc);
}

int b200_text_generate(b200_engine* e, const char* spec, const char* req, char** result_json_out) {
  ENTER();
  PyObject* p = NULL;
  int rc = call("text_generate", Py_BuildValue("(Lss)", e->handle, spec, req), &p);
  if (rc == 0 && result_json_out) *result_json_out = dup_str(p);
  Py_XDECREF(p);
  LEAVE(rc);
}

int b200_text_stream(b200_engine* e, const char* spec, const char* req, b200_chunk_cb cb, void* user) {
  ENTER();
  int rc = call("text_stream", Py_BuildValue("(LssKK)", e->handle, spec, req, (unsigned long long)(uintptr_t)cb,
                                             (unsigned long long)(uintptr_t)user), NULL);
  LEAVE(rc);
}

int b200_text_count_tokens(b200_engine* e, const char* spec, const char* req, int* tokens_out) {
  ENTER();
  PyObject* p = NULL;
  int rc = call("text_count_tokens", Py_BuildValue("(Lss)", e->handle, spec, req), &p);
  if (rc == 0 && tokens_out) *tokens_out = (int)PyLong_AsLong(p);
  Py_XDECREF(p);
  LEAVE(rc);
}

static uint8_t* dup_bytes(PyObject* b, Py_ssize_t* n) {
  char* data = NULL;
  PyBytes_AsStringAndSize(b, &data, n);
  uint8_t* out = (uint8_t*)malloc((size_t)(*n > 0 ? *n : 1));
  if (out && *n > 0) memcpy(out, data, (size_t)*n);
  return out;
}

int b200_image_generate(b200_engine* e, const char* spec, const char* req, b200_step_cb cb, void* user,
                        uint8_t** rgb_out, int* width, int* height, long long* seed) {
  ENTER();
  PyObject* p = NULL;
  int rc = call("image_generate", Py_BuildValue("(LssKK)", e->handle, spec, req, (unsigned long long)(uintptr_t)cb,
                                                (unsigned long long)(uintptr_t)user), &p);
  if (rc == 0) {   /* payload: (bytes, w, h, seed) */
    Py_ssize_t n = 0;
    if (rgb_out) *rgb_out = dup_bytes(PyTuple_GetItem(p, 0), &n);
    if (width) *width = (int)PyLong_AsLong(PyTuple_GetItem(p, 1));
    if (height) *height = (int)PyLong_AsLong(PyTuple_GetItem(p, 2));
    if (seed) *seed = PyLong_AsLongLong(PyTuple_GetItem(p, 3));
  }
  Py_XDECREF(p);
  LEAVE(rc);
}

int b200_video_generate(b200_engine* e, const char* spec, const char* req, b200_step_cb cb, void* user,
                        uint8_t** frames_out, int* frame_count, int* width, int* height, int* fps, long long* seed) {
  ENTER();
  PyObject* p = NULL;
  int rc = call("video_generate", Py_BuildValue("(LssKK)", e->handle, spec, req, (unsigned long long)(uintptr_t)cb,
                                                (unsigned long long)(uintptr_t)user), &p);
  if (rc == 0) {   /* payload: (bytes, count, w, h, fps, seed) */
    Py_ssize_t n = 0;
    if (frames_out) *frames_out = dup_bytes(PyTuple_GetItem(p, 0), &n);
    if (frame_count) *frame_count = (int)PyLong_AsLong(PyTuple_GetItem(p, 1));
    if (width) *width = (int)PyLong_AsLong(PyTuple_GetItem(p, 2));
    if (height) *height = (int)PyLong_AsLong(PyTuple_GetItem(p, 3));
    if (fps) *fps = (int)PyLong_AsLong(PyTuple_GetItem(p, 4));
    if (seed) *seed = PyLong_AsLongLong(PyTuple_GetItem(p, 5));
  }
  Py_XDECREF(p);
  LEAVE(rc);
}

int b200_transcribe(b200_engine* e, const char* spec, const char* req, const float* pcm, long long samples, int sample_rate,
                    char** result_json_out) {
  ENTER();
  PyObject* p = NULL;
  int rc = call("transcribe", Py_BuildValue("(Lssy#i)", e->handle, spec, req ? req : "{}", (const char*)pcm,
                                            (Py_ssize_t)(samples * (long long)sizeof(float)), sample_rate), &p);
  if (rc == 0 && result_json_out) *result_json_out = dup_str(p);
  Py_XDECREF(p);
  LEAVE(rc);
}

int b200_speak(b200_engine* e, const char* spec, const char* req, float** pcm_out, long long* samples_out, int* sample_rate_out) {
  ENTER();
  PyObject* p = NULL;
  int rc = call("speak", Py_BuildValue("(Lss)", e->handle, spec, req), &p);
  if (rc == 0) {   /* payload: (float32 bytes, sample rate) */
    Py_ssize_t n = 0;
    if (pcm_out) *pcm_out = (float*)dup_bytes(PyTuple_GetItem(p, 0), &n);
    if (samples_out) *samples_out = (long long)(n / (Py_ssize_t)sizeof(float));
    if (sample_rate_out) *sample_rate_out = (int)PyLong_AsLong(PyTuple_GetItem(p, 1));
  }
  Py_XDECREF(p);
  LEAVE(rc);
}

int b200_music(b200_engine* e, const char* spec, const char* req, float** pcm_out, long long* samples_out, int* sample_rate_out) {
  ENTER();
  PyObject* p = NULL;
  int rc = call("music", Py_BuildValue("(Lss)", e->handle, spec, req), &p);
  if (rc == 0) {   /* payload: (float32 bytes, sample rate) */
    Py_ssize_t n = 0;
    if (pcm_out) *pcm_out = (float*)dup_bytes(PyTuple_GetItem(p, 0), &n);
    if (samples_out) *samples_out = (long long)(n / (Py_ssize_t)sizeof(float));
    if (sample_rate_out) *sample_rate_out = (int)PyLong_AsLong(PyTuple_GetItem(p, 1));
  }
  Py_XDECREF(p);
  LEAVE(rc);
}

int b200_embed_text(b200_engine* e, const char* spec, const char* texts_json, float** out, int* count, int* dim) {
  ENTER();
  PyObject* p = NULL;
  int rc = call("embed_text", Py_BuildValue("(Lss)", e->handle, spec, texts_json), &p);
  if (rc == 0) {   /* payload: (float32 bytes, count, dim) */
    Py_ssize_t n = 0;
    if (out) *out = (float*)dup_bytes(PyTuple_GetItem(p, 0), &n);
    if (count) *count = (int)PyLong_AsLong(PyTuple_GetItem(p, 1));
    if (dim) *dim = (int)PyLong_AsLong(PyTuple_GetItem(p, 2));
  }
  Py_XDECREF(p);
  LEAVE(rc);
}

int b200_embed_image(b200_engine* e, const char* spec, const uint8_t* rgb, int width, int height, float** out, int* dim) {
  ENTER();
  PyObject* p = NULL;
  int rc = call("embed_image", Py_BuildValue("(Lsy#ii)", e->handle, spec, (const char*)rgb, (Py_ssize_t)width * height * 3,
                                             width, height), &p);
  if (rc == 0) {   /* payload: (float32 bytes, dim) */
    Py_ssize_t n = 0;
    if (out) *out = (float*)dup_bytes(PyTuple_GetItem(p, 0), &n);
    if (dim) *dim = (int)PyLong_AsLong(PyTuple_GetItem(p, 1));
  }
  Py_XDECREF(p);
  LEAVE(rc);
}

int b200_upscale(b200_engine* e, const char* spec, const char* req, const uint8_t* rgb, int width, int height,
                 uint8_t** rgb_out, int* width_out, int* height_out) {
  ENTER();
  PyObject* p = NULL;
  int rc = call("upscale", Py_BuildValue("(Lssy#ii)", e->handle, spec, req ? req : "{}", (const char*)rgb,
                                         (Py_ssize_t)width * height * 3, width, height), &p);
  if (rc == 0) {   /* payload: (bytes, w, h) */
    Py_ssize_t n = 0;
    if (rgb_out) *rgb_out = dup_bytes(PyTuple_GetItem(p, 0), &n);
    if (width_out) *width_out = (int)PyLong_AsLong(PyTuple_GetItem(p, 1));
    if (height_out) *height_out = (int)PyLong_AsLong(PyTuple_GetItem(p, 2));
  }
  Py_XDECREF(p);
  LEAVE(rc);
}

const char* b200_last_error(void) { return g_err; }
void b200_free(void* p) { free(p); }
const char* b200_version(void) { return "0.1.0"; }
