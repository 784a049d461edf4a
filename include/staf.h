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
 *   - with a caller-supplied list the pair vectors are plain Cartesian differences r_i - r_j (the
 *     reference subtracts fractional coordinates and skips the rint wrap, nn_nn_mlp.cu:847-853: the
 *     same vector up to rounding);
 *   - staf_compute_domain is an addition (see below).
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

/* Energy (0.5 * sum of the atomic energies of the nlocal owned atoms), forces f[nall*3] and virial[6]
 * (xx, yy, zz of W_ab = -sum g_a r_b; [3..5] = 0 as in staf_api.cpp:398-403) of one configuration.
 * x[nall*3] Cartesian, box[6] = Lx,xy,xz,Ly,yz,Lz, type[nall] 0-based species.
 * howmany == NULL: the library builds its own minimum-image neighbour list over the nlocal atoms
 * (nghost ignored, nall = nlocal), as the reference does (staf_api.cpp:211-212).
 * howmany[nlocal], with[nlocal*maxneigh] given (the LAMMPS contract, lammps/USER-STAF/pair_staf.cpp:180-233):
 * nall = nlocal + nghost, rows hold indices 0..nall-1, already cutoff-filtered and sorted by distance; ghosts
 * carry their periodic image, so no wrap is applied; forces are returned for the ghosts too and the caller
 * sums them onto their owners (reverse_comm).  Rows longer than the radial buffer are truncated
 * (staf_api.cpp:318-321).
 * Returns 0, or: -1 bad handle/argument/allocation, -3 nlocal <= 0, -7 zero box length, -8 species out of
 * range, -9 neighbour index out of range (all as staf_api.cpp:196-337), -11 radial buffer saturated,
 * -12 angular buffer saturated, -13 other device-side status, -14 CUDA error. */
int staf_compute(StafModel* m, int nlocal, int nghost, const double* x, const double* box, const int* type,
                 const int* howmany, const int* with, int maxneigh, double* e_rank, double* f, double* virial);

/* Addition (the reference has no such call): owned + ghost atoms WITHOUT a caller-built list.  The library
 * builds the neighbour list on the GPU over all nall = nlocal + nghost atoms with the minimum-image
 * convention of box[6]; only the nlocal owned atoms are centres.  For a spatial decomposition driver that
 * has no CPU neighbour list: every physical atom must appear at most once among owned + ghosts (any
 * periodic image of it will do), which holds for slab or brick domains wider than the cutoff.  Outputs and
 * return codes as staf_compute. */
int staf_compute_domain(StafModel* m, int nlocal, int nghost, const double* x, const double* box, const int* type,
                        double* e_rank, double* f, double* virial);

void staf_free(StafModel* m);

#ifdef __cplusplus
}
#endif
#endif /* STAF_H */
