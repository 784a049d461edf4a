// Driver around the reference's own native MLP evaluation (test infrastructure).
// Includes libstaf/src/mlp/staf_mlp_ort.cc from the reference tree as a
// translation unit (built without ONNX Runtime) and calls its public entry points
// staf_mlp_create / staf_mlp_eval (libstaf/include/staf_mlp.h:32-42), which run
// eval_type_native (staf_mlp_ort.cc:196-242) on mlp_type{k}.bin weights.
#include "staf_mlp.h"
#include <vector>

extern "C" int ref_mlp_eval(const char* model_dir, int precision, int n_type, const int* n_atoms, const int* n_af,
                            const void* af, void* energy, void* dE_daf) {
  StafMlp* mlp = staf_mlp_create(STAF_MLP_NATIVE, model_dir, precision, 0);
  if (!mlp) return -100;
  StafMlpEval io;
  io.n_type = n_type;
  io.n_atoms = n_atoms;
  io.n_af = n_af;
  io.af_f32 = precision == 0 ? (const float*)af : nullptr;
  io.af_f64 = precision == 1 ? (const double*)af : nullptr;
  io.energy_f32 = precision == 0 ? (float*)energy : nullptr;
  io.energy_f64 = precision == 1 ? (double*)energy : nullptr;
  io.dE_daf_f32 = precision == 0 ? (float*)dE_daf : nullptr;
  io.dE_daf_f64 = precision == 1 ? (double*)dE_daf : nullptr;
  int rc = staf_mlp_eval(mlp, &io);
  staf_mlp_destroy(mlp);
  return rc;
}
