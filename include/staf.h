/* staf.h - the libstaf C API, served by the B200 library (libstafb.so).
 *
 * Same names, argument order and meaning as the reference's libstaf/include/staf.h:12-61, so that
 * lammps/USER-STAF/pair_staf.cpp:95-117,233 and fix_staf.cpp:26-32 link against it unchanged.
 * Differences from the reference implementation (libstaf/src/staf_api.cpp):
 *   - all state lives in the StafModel handle (the reference keeps process-global statics in
 *     libstaf/vendor/jmd/nn_nn_mlp.cu:78-161 and chdir()s during initialisation);
 *   - the MLP runs on the GPU in the same stream as the descriptors (the reference copies the
 *     fingerprints to the host, evaluates ONNX Runtime / a CPU Dense loop and copies dE/dAF back:
 *     nn_nn_mlp.cu:657-768); mlp_backend is accepted and ignored, mlp_type{k}.bin is always read;
 *   - geometry, fingerprints and forces are computed in the precision of StafOptions.precision
 *     (the reference always uses double for those and the option only for the MLP);
 *   - the caller-supplied neighbour list (howmany != NULL, ghosts) is not built yet: staf_compute
 *     returns -10 for it; virial is returned as zeros.
 */
#ifndef STAF_H
#define STAF_H

#ifdef __cplusplus
extern "C" {
#endif

typedef struct StafModel StafModel;

typedef enum StafMlpBackend {
  STAF_MLP_ORT = 0,
  STAF_MLP_TF_C = 1,
  STAF_MLP_NATIVE = 2
} StafMlpBackend;

typedef struct StafOptions {
  StafMlpBackend mlp_backend; /* accepted for compatibility; the GPU MLP is always used */
  int device_id;              /* CUDA device for this rank */
  int precision;              /* 0 = float32, 1 = float64 */
  int reserved;
} StafOptions;

/* defaults: ORT, device 0, float32 (libstaf/src/staf_api.cpp:39-45) */
void staf_options_default(StafOptions* opt);

/* selects device_id % deviceCount; returns the id selected or -1 (staf_api.cpp:47-67) */
int staf_cuda_set_device(int device_id);

/* model_dir holds staf_jmd.cfg, type.dat, type{k}_alpha_2body.dat, type{k}_alpha_3body.dat,
 * type{k}_type_emb_{2b,3b}_sq.dat, type{k}_alpha_mu.dat and mlp_type{k}.bin (STAFMLP1).
 * Returns NULL on failure. */
StafModel* staf_load(const char* model_dir, const StafOptions* opt);

/* Energy (0.5 * sum of atomic energies), forces f[nall*3] and virial[6] of one configuration.
 * x[nall*3] Cartesian, box[6] = Lx,xy,xz,Ly,yz,Lz, type[nall] 0-based species.
 * howmany == NULL: the library builds its own minimum-image neighbour list over the nlocal atoms
 * (nghost ignored), as the reference does (staf_api.cpp:192-203).
 * Returns 0, or: -1 bad handle/allocation, -3 nlocal <= 0, -7 zero box length, -8 species out of range
 * (all as staf_api.cpp:196-337), -10 caller-supplied neighbour list not supported yet,
 * -11 radial buffer saturated, -12 angular buffer saturated, -13 other device-side status,
 * -14 CUDA error. */
int staf_compute(StafModel* m, int nlocal, int nghost, const double* x, const double* box, const int* type,
                 const int* howmany, const int* with, int maxneigh, double* e_rank, double* f, double* virial);

void staf_free(StafModel* m);

#ifdef __cplusplus
}
#endif
#endif /* STAF_H */
