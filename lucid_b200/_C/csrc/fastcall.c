/* CPython binding of the few liblucid_cuda entry points that decode-time dispatch calls once per
 * layer and forward, where the host, not the GPU, sets the pace: a ctypes call with some twenty
 * arguments costs about 3 us of marshalling, a METH_FASTCALL function a few tenths.  It plays the
 * part of the reference's pybind11 functions (lucid/_C/bindings/bind_quantized.cpp:17-27) for
 * these calls; every other entry point stays on ctypes, and so do these when this module has not
 * been built.
 *
 * The module does not link against the library: `bind(name, address)` hands it the address ctypes
 * resolved, and a call made before that raises.  Arguments are what the C declaration in
 * lucid_cuda.h takes, in its order: integers and raw addresses as Python ints, None for a null
 * pointer, floats as Python floats.  The result is the entry point's status code.  The calls only
 * enqueue work, so the GIL is kept.
 */
#define PY_SSIZE_T_CLEAN
#include <Python.h>
#include <stdint.h>
#include <string.h>

#include "lucid_cuda.h"

static __typeof__(lc_dynamic_linear_f32)* p_dynamic_linear_f32;
static __typeof__(lc_group_matmul_ex)* p_group_matmul_ex;
static __typeof__(lc_wo_linear_s8_ex)* p_wo_linear_s8_ex;
static __typeof__(lc_wo_swiglu_s8_ex)* p_wo_swiglu_s8_ex;

static inline int64_t as_int(PyObject* o) {
  if (o == Py_None) return 0;
  return (int64_t)PyLong_AsUnsignedLongLongMask(o);  /* addresses above 2^63 and negative values alike */
}

static PyObject* finish(int32_t rc) {
  if (PyErr_Occurred()) return NULL;  /* an argument was not an int / float: the call was made with zeros */
  return PyLong_FromLong(rc);
}

static PyObject* unbound(const char* name, Py_ssize_t expected, Py_ssize_t got, int bound) {
  if (!bound) return PyErr_Format(PyExc_RuntimeError, "%s: no address bound", name);
  return PyErr_Format(PyExc_TypeError, "%s takes %zd arguments, got %zd", name, expected, got);
}

/* every argument is checked before the call: a conversion error must not launch anything */
static int convert(PyObject* const* args, Py_ssize_t n, int float_at, int64_t* iv, double* fv) {
  for (Py_ssize_t i = 0; i < n; ++i) {
    if (i == float_at) {
      *fv = PyFloat_AsDouble(args[i]);
      iv[i] = 0;
    } else {
      iv[i] = as_int(args[i]);
    }
    if (PyErr_Occurred()) return 0;
  }
  return 1;
}

#define A(i) iv[i]
#define P(i) ((void*)(uintptr_t)iv[i])

static PyObject* f_dynamic_linear_f32(PyObject* self, PyObject* const* args, Py_ssize_t n) {
  int64_t iv[23];
  double eps = 0.0;
  if (n != 23 || !p_dynamic_linear_f32) return unbound("dynamic_linear_f32", 23, n, p_dynamic_linear_f32 != NULL);
  if (!convert(args, n, 8, iv, &eps)) return NULL;
  return finish(p_dynamic_linear_f32(P(0), A(1), A(2), A(3), (int32_t)A(4), (int32_t)A(5), (int32_t)A(6), (int32_t)A(7),
                                     (float)eps, P(9), A(10), A(11), P(12), P(13), P(14), P(15), (int32_t)A(16), A(17),
                                     P(18), A(19), (int32_t)A(20), P(21), P(22)));
}

static PyObject* f_group_matmul_ex(PyObject* self, PyObject* const* args, Py_ssize_t n) {
  int64_t iv[15];
  double unused = 0.0;
  if (n != 15 || !p_group_matmul_ex) return unbound("group_matmul_ex", 15, n, p_group_matmul_ex != NULL);
  if (!convert(args, n, -1, iv, &unused)) return NULL;
  return finish(p_group_matmul_ex(P(0), (int32_t)A(1), A(2), A(3), P(4), P(5), P(6), A(7), (int32_t)A(8), (int32_t)A(9),
                                  P(10), (int32_t)A(11), P(12), A(13), P(14)));
}

static PyObject* f_wo_linear_s8_ex(PyObject* self, PyObject* const* args, Py_ssize_t n) {
  int64_t iv[21];
  double unused = 0.0;
  if (n != 21 || !p_wo_linear_s8_ex) return unbound("wo_linear_s8_ex", 21, n, p_wo_linear_s8_ex != NULL);
  if (!convert(args, n, -1, iv, &unused)) return NULL;
  return finish(p_wo_linear_s8_ex(P(0), (int32_t)A(1), A(2), A(3), A(4), P(5), A(6), A(7), P(8), P(9), (int32_t)A(10),
                                  P(11), P(12), (int32_t)A(13), (int32_t)A(14), P(15), A(16), (int32_t)A(17), P(18),
                                  A(19), P(20)));
}

static PyObject* f_wo_swiglu_s8_ex(PyObject* self, PyObject* const* args, Py_ssize_t n) {
  int64_t iv[16];
  double unused = 0.0;
  if (n != 16 || !p_wo_swiglu_s8_ex) return unbound("wo_swiglu_s8_ex", 16, n, p_wo_swiglu_s8_ex != NULL);
  if (!convert(args, n, -1, iv, &unused)) return NULL;
  return finish(p_wo_swiglu_s8_ex(P(0), (int32_t)A(1), A(2), A(3), A(4), P(5), A(6), A(7), P(8), P(9), P(10), A(11),
                                  (int32_t)A(12), P(13), A(14), P(15)));
}

static PyObject* f_bind(PyObject* self, PyObject* args) {
  const char* name;
  unsigned long long address;
  if (!PyArg_ParseTuple(args, "sK", &name, &address)) return NULL;
  void* p = (void*)(uintptr_t)address;
  if (!strcmp(name, "lc_dynamic_linear_f32")) p_dynamic_linear_f32 = (__typeof__(p_dynamic_linear_f32))p;
  else if (!strcmp(name, "lc_group_matmul_ex")) p_group_matmul_ex = (__typeof__(p_group_matmul_ex))p;
  else if (!strcmp(name, "lc_wo_linear_s8_ex")) p_wo_linear_s8_ex = (__typeof__(p_wo_linear_s8_ex))p;
  else if (!strcmp(name, "lc_wo_swiglu_s8_ex")) p_wo_swiglu_s8_ex = (__typeof__(p_wo_swiglu_s8_ex))p;
  else return PyErr_Format(PyExc_KeyError, "no fast binding for %s", name);
  Py_RETURN_NONE;
}

static PyMethodDef methods[] = {
    {"bind", f_bind, METH_VARARGS, "bind(name, address): the address of a liblucid_cuda entry point"},
    {"dynamic_linear_f32", (PyCFunction)(void (*)(void))f_dynamic_linear_f32, METH_FASTCALL, "lc_dynamic_linear_f32"},
    {"group_matmul_ex", (PyCFunction)(void (*)(void))f_group_matmul_ex, METH_FASTCALL, "lc_group_matmul_ex"},
    {"wo_linear_s8_ex", (PyCFunction)(void (*)(void))f_wo_linear_s8_ex, METH_FASTCALL, "lc_wo_linear_s8_ex"},
    {"wo_swiglu_s8_ex", (PyCFunction)(void (*)(void))f_wo_swiglu_s8_ex, METH_FASTCALL, "lc_wo_swiglu_s8_ex"},
    {NULL, NULL, 0, NULL}};

static struct PyModuleDef module = {PyModuleDef_HEAD_INIT, "_fastcall", "low-overhead calls into liblucid_cuda", -1, methods};

PyMODINIT_FUNC PyInit__fastcall(void) { return PyModule_Create(&module); }
