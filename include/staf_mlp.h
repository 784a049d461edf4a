/* staf_mlp.h - the pluggable-MLP C API of libstaf, served by the B200 library (libstafb.so).
 *
 * Same names, argument order and meaning as the reference's libstaf/include/staf_mlp.h:17-42: atomic
 * fingerprints in, energy and dE/dAF out, host arrays.  Convention (staf_mlp.h:10-15 of the reference):
 * energy = 0.5 * sum(atomic energies); dE_daf = d(sum of atomic energies)/dAF; the network input is
 * log(AF + 1e-3) - mu (libstaf/src/mlp/staf_mlp_ort.cc:196-242).
 * Differences from the reference implementation: the Dense layers run on the GPU (the same kernel that serves
 * staf_compute); `backend` is accepted and ignored, mlp_type{k}.bin is always read; model_dir must be a complete
 * model directory as for staf_load (the descriptor files are read too, because one loader serves both APIs).
 */
#ifndef STAF_MLP_H
#define STAF_MLP_H

#ifdef __cplusplus
extern "C" {
#endif

#include "staf.h"

typedef struct StafMlp StafMlp;

typedef struct StafMlpEval {
  int n_type;
  const int* n_atoms; /* [n_type] */
  const int* n_af;    /* [n_type] */
  /* Packed AF per type: type0 atoms, then type1, ... row-major [n_atoms_k, n_af_k] */
  const float* af_f32;
  const double* af_f64;
  float* energy_f32; /* [1] total for all types */
  double* energy_f64;
  float* dE_daf_f32; /* packed like af */
  double* dE_daf_f64;
} StafMlpEval;

/* precision: 0 = float32, 1 = float64.  Returns NULL on failure. */
StafMlp* staf_mlp_create(StafMlpBackend backend, const char* model_dir, int precision, int device_id);
/* The arrays of the created precision are used (af_f32/energy_f32/dE_daf_f32 or the _f64 ones).
 * Returns 0, or -1 bad handle/argument/allocation, -2 n_type or n_af do not match the model, -13 device-side
 * status, -14 CUDA error. */
int staf_mlp_eval(StafMlp* mlp, StafMlpEval* io);
void staf_mlp_destroy(StafMlp* mlp);

/* Number of loaded type nets (after create). */
int staf_mlp_ntypes(const StafMlp* mlp);
int staf_mlp_n_af(const StafMlp* mlp, int type);
/* 0 = float32, 1 = float64 (matches create precision). */
int staf_mlp_precision(const StafMlp* mlp);

#ifdef __cplusplus
}
#endif
#endif /* STAF_MLP_H */
