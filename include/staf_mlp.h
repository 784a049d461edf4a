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
  int n_type;         /* number of species */
  const int* n_atoms; /* atoms of every species, n_type entries */
  const int* n_af;    /* fingerprints per atom of every species, n_type entries */
  /* Fingerprints of all atoms in one array: the atoms of species 0 first, then species 1 ...; inside a species
   * one row of n_af[k] values per atom.  Only the array of the handle's precision is read. */
  const float* af_f32;
  const double* af_f64;
  /* Out: one value, half the sum of the atomic energies over all species. */
  float* energy_f32;
  double* energy_f64;
  /* Out: derivative of the sum of the atomic energies with respect to every fingerprint, laid out as af. */
  float* dE_daf_f32;
  double* dE_daf_f64;
} StafMlpEval;

/* precision: 0 for float32, 1 for float64.  NULL when the model cannot be loaded. */
StafMlp* staf_mlp_create(StafMlpBackend backend, const char* model_dir, int precision, int device_id);
/* Returns 0, or -1 bad handle/argument/allocation, -2 n_type or n_af do not match the model, -13 device-side
 * status, -14 CUDA error. */
int staf_mlp_eval(StafMlp* mlp, StafMlpEval* io);
void staf_mlp_destroy(StafMlp* mlp);

/* what was loaded: species count, fingerprints per atom of a species, precision (0 / 1 as in create) */
int staf_mlp_ntypes(const StafMlp* mlp);
int staf_mlp_n_af(const StafMlp* mlp, int type);
int staf_mlp_precision(const StafMlp* mlp);

#ifdef __cplusplus
}
#endif
#endif /* STAF_MLP_H */
