/* stafb.h - C ABI of the B200 (sm_100a) implementation of the STAF descriptor / fingerprint /
 * force / gradient hot path.
 *
 * Every entry point takes plain pointers and sizes.  Pointers named *_d are DEVICE pointers
 * unless the function name ends in _host.  `real` tensors are float or double according to
 * the dtype the context was created with (the reference builds two op trees, ops_float and
 * ops_double, from one source: STAF/include/staf_real.h:21-37).  All index tensors are int32.
 * `stream` is a cudaStream_t passed as void* (NULL = default stream).  Calls are asynchronous
 * on that stream unless stated otherwise.  No entry point ever terminates the process: where
 * the reference calls exit() the library returns / records a status code.
 *
 * Paths in the comments are relative to the reference project root.
 */
#ifndef STAFB_H
#define STAFB_H

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

#define STAFB_OK 0
#define STAFB_ERR_RADIAL_OVERFLOW 1  /* an atom has more than radial_buffer neighbours
                                        (reference: printf + exit(0), descriptor_builder/reforce.cc:324-340) */
#define STAFB_ERR_ANGULAR_OVERFLOW 2 /* m(m-1)/2 > angular_buffer (reference: silently dropped by the kernels,
                                        sys.exit in staf_train.py:709-714) */
#define STAFB_ERR_CELL_OVERFLOW 3    /* a cell holds more than MAX_PARTICLE_CELLS atoms (reference: silently
                                        dropped, descriptor_builder/celle_gpu.cu.cc:197-200) */
#define STAFB_ERR_BAD_BOX 4          /* zero box length (reference: libstaf/src/staf_api.cpp returns -7) */
#define STAFB_ERR_INVALID 5          /* bad argument */
#define STAFB_ERR_CUDA 6             /* a CUDA runtime call failed; see stafb_last_cuda_error() */
#define STAFB_ERR_CAPACITY 7         /* nf or N larger than what the context was created for */
#define STAFB_ERR_NONFINITE 8        /* non-finite energy */
#define STAFB_ERR_PEER_TIMEOUT 9     /* stafb_allreduce_adam, stafb_halo_*: a peer rank did not publish in time */
#define STAFB_ERR_STAGE_TIMEOUT 10   /* a kernel gave up waiting for its own asynchronous copy into shared memory */

#define STAFB_F32 0
#define STAFB_F64 1
#define STAFB_MAX_TYPES 4
#define STAFB_MAX_DENSE 6

typedef struct stafb_ctx stafb_ctx;
typedef struct stafb_model stafb_model;

/* ---- context ------------------------------------------------------------------------------
 * Replaces op ConstructDescriptorsLight (descriptor_builder/reforce.cc:182-238): stores the
 * cutoffs and buffer sizes, computes the repulsive-core coefficients (fill_repulsion,
 * reforce.cc:101-125; the cutoff_curve.dat side effect is dropped) and allocates the per-device
 * scratch (cells, neighbour rows) for max_batch frames of n_max atoms on the CURRENT device.
 * State lives in the handle, not in process globals. */
int stafb_create(stafb_ctx** out, int dtype, double radial_cutoff, double rs, double ra, int radial_buffer,
                 int angular_buffer, int n_max, int max_batch);
void stafb_destroy(stafb_ctx* ctx);
/* Synchronises `stream` and returns the first status recorded by device code since the last
 * call (STAFB_OK if none), then clears it. */
int stafb_status(stafb_ctx* ctx, void* stream);
const char* stafb_strerror(int status);
const char* stafb_last_cuda_error(void);
/* coefficients A, B, C and the powers (1, -30) of the repulsive core, as doubles */
void stafb_core_coefficients(const stafb_ctx* ctx, double out5[5]);

/* ---- the reference's operators, one function each ------------------------------------------
 * Shapes: nf frames, N atoms, Nl atoms of the central species, nr = radial_buffer,
 * na = angular_buffer, nt species, C = nt(nt+1)/2, Fr / Fa radial / angular fingerprints. */

/* ComputeDescriptorsLight (descriptor_builder/reforce.cc:241-252,262-444).
 * positions[nf,3N] Cartesian, boxer[nf,6] = Lx,xy,xz,Ly,yz,Lz ->
 * raddescr[nf,N,nr] angdescr[nf,N,na] des3bsupp[nf,N,nr] intmap2b[nf,N,nr+1] intmap3b[nf,N,2na]
 * der2b[nf,N,3,nr] der3b[nf,N,3,2na] der3bsupp[nf,N,3,nr] numtriplet[nf,N].
 * angdescr, intmap3b and der3b may all be NULL (the three angular tensors are then not produced).
 * Padded slots, which the reference leaves uninitialised in the float tensors, are zero. */
int stafb_compute_descriptors_light(stafb_ctx* ctx, void* stream, const void* positions_d, const void* boxer_d,
                                    int nf, int N, void* raddescr_d, void* angdescr_d, void* des3bsupp_d,
                                    int* intmap2b_d, int* intmap3b_d, void* der2b_d, void* der3b_d,
                                    void* der3bsupp_d, int* numtriplet_d);

/* ComputeDescriptorsLight for callers that must not allocate.  No counterpart in the reference.
 * stafb_create() obtains the neighbour-list scratch with cudaMalloc; some callers cannot do that where
 * they need the descriptors (an op callback whose device memory belongs to the host framework's
 * allocator, a plug-in entered while another library holds the allocator lock, a process with a fixed
 * memory budget).  This entry point takes no handle and allocates nothing: the scratch is a fixed array
 * inside the library image (stafb_noalloc_scratch_bytes() bytes, about 3.3 MB, held by every GPU that
 * loads the library until the process exits).  Limits: nf <= 16, nf*N <= 1024 atoms, radial_buffer <= 64;
 * larger requests return STAFB_ERR_CAPACITY and print the limits.  The first call on a device looks up
 * the array's device address (cudaGetSymbolAddress); make that first call outside any stream capture.
 * All calls share the array: calls that overlap on one GPU race, so serialise them (one stream).  Outputs
 * and their optional/NULL rules are those of stafb_compute_descriptors_light; status_out_d (device int)
 * receives the status word (STAFB_OK, STAFB_ERR_RADIAL_OVERFLOW, ...) on the stream.  There is no handle, so
 * that word is the ONLY report of a saturated radial or angular buffer, a bad box or a cell overflow: with
 * status_out_d == NULL such a call returns STAFB_OK and truncated rows, unnoticed - pass it. */
int stafb_compute_descriptors_light_noalloc(int dtype, double radial_cutoff, double rs, double ra, int radial_buffer,
                                            int angular_buffer, void* stream, const void* positions_d,
                                            const void* boxer_d, int nf, int N, void* raddescr_d, void* angdescr_d,
                                            void* des3bsupp_d, int* intmap2b_d, int* intmap3b_d, void* der2b_d,
                                            void* der3b_d, void* der3bsupp_d, int* numtriplet_d, int* status_out_d);
size_t stafb_noalloc_scratch_bytes(void);

/* ComputeSortProj (fingerprint/rad/reforce.cc:13-19) -> two_body_afs[nf,Nl,Fr] */
int stafb_compute_sort_proj(stafb_ctx* ctx, void* stream, const void* radial_descriptor_d,
                            const int* interaction_map_rad_d, const void* alpha2b_d, const void* type_emb2b_sq_d,
                            const int* type_map_d, int nf, int Nl, int nt, int Fr, void* two_body_afs_d);

/* ComputeSortProj3body (fingerprint/ang/reforce.cc:15-24) -> three_body_afs[nf,Nl,Fa].
 * radial_descriptor is des3bsupp (source_routine/physics_layer_mod.py:40). */
int stafb_compute_sort_proj3body(stafb_ctx* ctx, void* stream, const void* angular_descriptor_d,
                                 const void* radial_descriptor_d, const int* interaction_map_angular_d,
                                 const int* interaction_map_rad_d, const void* alpha3b_d,
                                 const void* type_emb3b_sq_d, const int* type_map_d, const int* num_triplet_d, int nf,
                                 int Nl, int nt, int Fa, void* three_body_afs_d);

/* InitForceRadial / InitForceTripl / InitGradForceRadial / InitGradForceTripl
 * (force/rad/reforce.cc:13-36 and siblings) chose a CUDA block size from the buffer size; the
 * library needs no such state.  Kept so that callers can keep calling them: returns 0. */
int stafb_init_force_radial(int buffdim);
int stafb_init_force_tripl(int buffdim);
int stafb_init_grad_force_radial(int buffdim);
int stafb_init_grad_force_tripl(int buffdim);

/* ComputeForceRadial (force/rad/reforce.cc:39-49) -> force[nf,3N] (zero-filled, then this
 * species' contribution).  tipos[nt] and actual_type[1] are device tensors as in the op. */
int stafb_compute_force_radial(stafb_ctx* ctx, void* stream, const void* netderiv_d,
                               const void* descriptor_derivative_rad_d, const int* interaction_map_rad_d,
                               const void* radial_descriptor_d, const void* alpha2b_d, const void* type_emb2b_sq_d,
                               const int* type_map_d, const int* tipos_d, const int* actual_type_d, int nf, int Nl,
                               int N, int nt, int Fr, void* force_d);

/* ComputeForceTripl (force/ang/reforce.cc:44-58) -> force[nf,3N] */
int stafb_compute_force_tripl(stafb_ctx* ctx, void* stream, const void* netderiv_d, const void* radial_descriptor_d,
                              const void* angular_descriptor_d, const void* descriptor_derivative_rad_d,
                              const void* descriptor_derivative_ang_d, const int* interaction_map_rad_d,
                              const int* interaction_map_ang_d, const void* alpha3b_d, const void* type_emb3b_sq_d,
                              const int* type_map_d, const int* tipos_d, const int* actual_type_d,
                              const int* num_triplets_d, int nf, int Nl, int N, int nt, int Fa, void* force_d);

/* ComputeTwoBodyParGrad (grad_finger/rad/reforce.cc:14-22) -> nextgrad_alpha2b[nt,Fr], nextgrad_emb2b[nt,Fr] */
int stafb_compute_two_body_par_grad(stafb_ctx* ctx, void* stream, const void* prev_grad_d,
                                    const void* radial_descriptor_d, const int* interaction_map_rad_d,
                                    const void* alpha2b_d, const void* type_emb2b_sq_d, const int* type_map_d, int nf,
                                    int Nl, int nt, int Fr, void* nextgrad_alpha2b_d, void* nextgrad_emb2b_d);

/* ComputeSortProj3bodyGrad (grad_finger/ang/reforce.cc:12-23) -> alphagrad3body[C,3Fa] and
 * nextgrad_emb3b[C,Fa], which the reference never accumulates into: written as zeros. */
int stafb_compute_sort_proj3body_grad(stafb_ctx* ctx, void* stream, const void* previous_gradient_d,
                                      const void* angular_descriptors_d, const void* radial_descriptors_d,
                                      const int* intmap3b_d, const int* intmap2b_d, const void* alpha3b_d,
                                      const void* type_emb3b_sq_d, const int* type_map_d, const int* num_triplets_d,
                                      int nf, int Nl, int nt, int Fa, void* alphagrad3body_d, void* nextgrad_emb3b_d);

/* ComputeForceRadialGrad (grad_force/rad/reforce.cc:42-55) -> gradnet[nf,Nl,Fr], grad_alpha2b[nt,Fr], grad_emb2b[nt,Fr] */
int stafb_compute_force_radial_grad(stafb_ctx* ctx, void* stream, const void* prevgrad_d, const void* netderiv_d,
                                    const void* descriptor_derivative_rad_d, const int* interaction_map_rad_d,
                                    const void* radial_descriptor_d, const void* alpha2b_d,
                                    const void* type_emb2b_sq_d, const int* type_map_d, const int* tipos_d,
                                    const int* actual_type_d, int nf, int Nl, int N, int nt, int Fr, void* gradnet_d,
                                    void* grad_alpha2b_d, void* grad_emb2b_d);

/* ComputeForceTriplGrad (grad_force/ang/reforce.cc:39-56) -> gradnet[nf,Nl,Fa], gradalpha[C,3Fa],
 * gradck[C,Fa] (never written by the reference: zeros). */
int stafb_compute_force_tripl_grad(stafb_ctx* ctx, void* stream, const void* prevgrad_d, const void* netderiv_d,
                                   const void* radial_descriptor_d, const void* angular_descriptor_d,
                                   const void* descriptor_derivative_rad_d, const void* descriptor_derivative_ang_d,
                                   const int* interaction_map_rad_d, const int* interaction_map_ang_d,
                                   const void* alpha3b_d, const void* type_emb3b_sq_d, const int* type_map_d,
                                   const int* tipos_d, const int* actual_type_d, const int* num_triplets_d, int nf,
                                   int Nl, int N, int nt, int Fa, void* gradnet_d, void* gradalpha_d, void* gradck_d);

/* ComputeForceRadialVirial (force/rad/reforce.cc:133-146): ComputeForceRadial plus virial[nf,9] (row-major 3x3,
 * W_ab = -sum g_a r_b with r = r_i - r_j under the minimum image of box; zero-filled, then this species'
 * contribution).  pos[nf,3N] Cartesian, box[nf,6]. */
int stafb_compute_force_radial_virial(stafb_ctx* ctx, void* stream, const void* netderiv_d,
                                      const void* descriptor_derivative_rad_d, const int* interaction_map_rad_d,
                                      const void* radial_descriptor_d, const void* alpha2b_d,
                                      const void* type_emb2b_sq_d, const int* type_map_d, const int* tipos_d,
                                      const int* actual_type_d, const void* pos_d, const void* box_d, int nf, int Nl,
                                      int N, int nt, int Fr, void* force_d, void* virial_d);

/* ComputeForceTriplVirial (force/ang/reforce.cc:159-176) */
int stafb_compute_force_tripl_virial(stafb_ctx* ctx, void* stream, const void* netderiv_d,
                                     const void* radial_descriptor_d, const void* angular_descriptor_d,
                                     const void* descriptor_derivative_rad_d, const void* descriptor_derivative_ang_d,
                                     const int* interaction_map_rad_d, const int* interaction_map_ang_d,
                                     const void* alpha3b_d, const void* type_emb3b_sq_d, const int* type_map_d,
                                     const int* tipos_d, const int* actual_type_d, const int* num_triplets_d,
                                     const void* pos_d, const void* box_d, int nf, int Nl, int N, int nt, int Fa,
                                     void* force_d, void* virial_d);

/* ComputeForceRadialVirialGrad (grad_force/rad/reforce.cc:160-176): backward of ComputeForceRadialVirial for the
 * cotangents prevgrad[nf,3N] on the force and prevgrad_virial[nf,9] on the virial. */
int stafb_compute_force_radial_virial_grad(stafb_ctx* ctx, void* stream, const void* prevgrad_d,
                                           const void* prevgrad_virial_d, const void* netderiv_d,
                                           const void* descriptor_derivative_rad_d, const int* interaction_map_rad_d,
                                           const void* radial_descriptor_d, const void* alpha2b_d,
                                           const void* type_emb2b_sq_d, const int* type_map_d, const int* tipos_d,
                                           const int* actual_type_d, const void* pos_d, const void* box_d, int nf,
                                           int Nl, int N, int nt, int Fr, void* gradnet_d, void* grad_alpha2b_d,
                                           void* grad_emb2b_d);

/* ComputeForceTriplVirialGrad (grad_force/ang/reforce.cc:186-206); gradck is zeros like in ComputeForceTriplGrad */
int stafb_compute_force_tripl_virial_grad(stafb_ctx* ctx, void* stream, const void* prevgrad_d,
                                          const void* prevgrad_virial_d, const void* netderiv_d,
                                          const void* radial_descriptor_d, const void* angular_descriptor_d,
                                          const void* descriptor_derivative_rad_d,
                                          const void* descriptor_derivative_ang_d, const int* interaction_map_rad_d,
                                          const int* interaction_map_ang_d, const void* alpha3b_d,
                                          const void* type_emb3b_sq_d, const int* type_map_d, const int* tipos_d,
                                          const int* actual_type_d, const int* num_triplets_d, const void* pos_d,
                                          const void* box_d, int nf, int Nl, int N, int nt, int Fa, void* gradnet_d,
                                          void* gradalpha_d, void* gradck_d);

/* ---- fused path ----------------------------------------------------------------------------
 * One model = nt per-species blocks of trained parameters in ONE flat buffer `theta`
 *     alpha2b[nt,Fr_t] | alpha3b[C,3Fa_t] | mu[Fr_t+Fa_t] | W0[in,out] b0 | W1 b1 | ...   (t = 0..nt-1)
 * and the squared type embeddings (never trained: staf_models/staf_model.py:225-253) in `emb`
 *     e2[nt,Fr_t] | e3[C,Fa_t]                                                                (t = 0..nt-1).
 * shape_desc = int32[20]: nt, tipos[4], Fr[4], Fa[4], n_dense, width[6] (width[n_dense-1] == 1; hidden
 * layers are tanh, the output layer is linear).  Atoms are species-sorted (staf_train.py:217-224). */
int stafb_model_create(stafb_ctx* ctx, const int* shape_desc, stafb_model** out);
void stafb_model_destroy(stafb_model* m);
int stafb_model_n_params(const stafb_model* m);
int stafb_model_n_emb(const stafb_model* m);
/* offsets of species t: a2, a3, mu, w (into theta), emb (into emb), block size */
void stafb_model_offsets(const stafb_model* m, int t, int out6[6]);

/* How the MLP kernels of this model were configured (no reference counterpart; for tests and diagnostics):
 * out4 = { staging mode of the Dense layers in shared memory (2: all layers at kernel start, 1: one layer at a
 * time, 0: none, weights read from global memory), atoms per thread group (a block owns 8x that many atoms),
 * dynamic shared memory of the forward kernel, of the backward kernel (bytes) }.  The mode follows from the
 * layer sizes; the environment variables STAFB_MLP_STAGE / STAFB_MLP_AW, read by stafb_model_create,
 * override it. */
void stafb_model_mlp_config(const stafb_model* m, int out4[4]);
/* The other arm of the MLP kernels (fp32 models only, selected with STAFB_MLP_MMA=1 in the environment of
 * stafb_model_create): every dense product as mma.sync on the tensor cores - TF32 operands split in two, three
 * products per tile, the main product accumulated outside the unit: fp32 accuracy.  On B200 it is slower than
 * the FMA kernels (the legacy mma.sync path issues about one m16n8k8 per 30 cycles per SM), so it is off by
 * default.  out4 = { 1 if in use, its warps per block (a block owns 16 atoms; STAFB_MLP_MMA_NW: 1, 2, 4, 8),
 * 0, dynamic shared memory of the backward kernel }. */
void stafb_model_mlp_mma_config(const stafb_model* m, int out4[4]);

/* Energy and forces of nf frames (staf_models/staf_model.py:174-211; inference convention
 * staf_models/staf_model_inference_full.py:118-119 when per_atom_energy == 0):
 * energy[nf] = 0.5*mean_i e_i (per_atom_energy) or 0.5*sum_i e_i; force[nf,3N]. */
int stafb_energy_force(stafb_ctx* ctx, stafb_model* m, void* stream, const void* positions_d, const void* boxer_d,
                       int nf, const void* theta_d, const void* emb_d, int per_atom_energy, void* energy_d,
                       void* force_d);

/* New species counts for an existing model (same parameter layout): atoms per species may change from call
 * to call as long as their sum stays within the n_max the context was created with.  An MD driver whose
 * owned atoms migrate between domains (lammps/USER-STAF/pair_staf.cpp:180-256 rebuilds its arrays every step)
 * calls this instead of recreating the model. */
int stafb_model_set_counts(stafb_model* m, const int* tipos);

/* Energy and forces of ONE frame in which only the first N atoms (the model's species-sorted atoms) are
 * centres and the remaining nall-N atoms are ghosts: they act as neighbours and receive forces but
 * contribute no atomic energy - the owned/ghost contract of libstaf's staf_compute
 * (libstaf/include/staf.h:38-59, libstaf/src/staf_api.cpp:230-347).  type_map[nall] gives the species of
 * every atom (the ghosts are not species-sorted).  energy[1] = 0.5*sum over the centres; force[nall,3].
 *   howmany == NULL: the library builds the neighbour list over all nall atoms with the minimum-image
 *     convention of boxer[6] (every physical atom must appear at most once among owned + ghosts);
 *   howmany[N], with[N, radial_buffer] given: rows are taken as they are (cutoff-filtered and
 *     distance-sorted by the caller, indices 0..nall-1), vectors are plain Cartesian differences because the
 *     ghosts carry their periodic image (libstaf/vendor/jmd/nn_nn_mlp.cu:847-853); boxer may be NULL. */
int stafb_energy_force_domain(stafb_ctx* ctx, stafb_model* m, void* stream, const void* positions_d,
                              const void* boxer_d, int nall, const int* type_map_d, const int* howmany_d,
                              const int* with_d, const void* theta_d, const void* emb_d, void* energy_d,
                              void* force_d, void* virial_d /* [9] or NULL */);

/* stafb_energy_force plus the 3x3 virial W_ab = -sum g_a r_b of every frame (virial[nf,9], row-major), the sum
 * of what ComputeForceRadialVirial and ComputeForceTriplVirial return over all central species
 * (force/rad/reforce.cc:133-146, force/ang/reforce.cc:159-176; staf_models/staf_model_inference_full.py:89-144). */
int stafb_energy_force_virial(stafb_ctx* ctx, stafb_model* m, void* stream, const void* positions_d,
                              const void* boxer_d, int nf, const void* theta_d, const void* emb_d,
                              int per_atom_energy, void* energy_d, void* force_d, void* virial_d);

/* One energy+force training evaluation (full_train_e_f, staf_models/staf_model.py:168-258, without
 * the optimizer update): loss = pe*L(E,e_label) + pb*sum(alpha*[alpha>alpha_bound]) + pf*L(F,f_label),
 * L = Keras Huber(delta=1, mean) if loss_kind == 0 else MSE.  Writes losses[4] (double: loss, loss_e,
 * loss_bound, loss_f) and grad[n_params] = dloss/dtheta.  energy_d / force_d may be NULL. */
int stafb_train_step(stafb_ctx* ctx, stafb_model* m, void* stream, const void* positions_d, const void* boxer_d,
                     int nf, const void* theta_d, const void* emb_d, const void* e_label_d, const void* f_label_d,
                     double pe, double pf, double pb, double alpha_bound, int loss_kind, double* losses_d,
                     void* grad_d, void* energy_d, void* force_d);

/* The same with the virial term of full_train_e_f_v (STAF/staf_models/staf_model.py:313-384): v_label_d[nf,9]
 * total virials, loss = pe*loss_e + pb*loss_bound + pf*loss_f + pv*loss_v with loss_v the mean of L(W - W_label)
 * over [nf,9]; W = -sum f_a r_b over the pairs as the ...Virial force operators define it.
 * losses_d[5] = loss, loss_e, loss_bound, loss_f, loss_v; virial_d[nf,9] (optional) receives W. */
int stafb_train_step_virial(stafb_ctx* ctx, stafb_model* m, void* stream, const void* positions_d,
                            const void* boxer_d, int nf, const void* theta_d, const void* emb_d,
                            const void* e_label_d, const void* f_label_d, const void* v_label_d, double pe, double pf,
                            double pv, double pb, double alpha_bound, int loss_kind, double* losses_d, void* grad_d,
                            void* energy_d, void* force_d, void* virial_d);

/* stafb_train_step in two parts, for callers that know the next batch early (the reference's training loop
 * prefetches its batches in a thread, STAF/staf_train.py:678-755).  The neighbour rows of a batch depend on its
 * positions and boxes only - not on theta - so _prefetch may run on ANOTHER stream while the previous step, the
 * gradient all-reduce or the optimiser update still occupy `stream`; the model keeps two sets of rows (slot 0, 1,
 * allocated on first use).  stafb_train_step_prefetched then runs the rest of the step (fingerprints, network,
 * forces, loss, backward) on the rows of `slot`.  Ordering is the caller's: the rest of the step must wait for
 * the prefetch of its slot (an event), and a slot must not be prefetched again before the step that reads it has
 * finished.  Results are identical to stafb_train_step's. */
int stafb_descriptors_prefetch(stafb_ctx* ctx, stafb_model* m, void* stream, const void* positions_d,
                               const void* boxer_d, int nf, int slot);
int stafb_train_step_prefetched(stafb_ctx* ctx, stafb_model* m, void* stream, int slot, int nf, const void* theta_d,
                                const void* emb_d, const void* e_label_d, const void* f_label_d, double pe,
                                double pf, double pb, double alpha_bound, int loss_kind, double* losses_d,
                                void* grad_d, void* energy_d, void* force_d);

/* Adam update of theta in place (Keras Adam, epsilon default 1e-7: optimizer_learning_rate_utility.py:64-68):
 * g = grad*grad_scale; m,v moments; step counts from 1. */
int stafb_adam_step(stafb_ctx* ctx, void* stream, void* theta_d, const void* grad_d, void* m_d, void* v_d, int n,
                    double lr, double beta1, double beta2, double eps, int step, double grad_scale);

/* Adam with the step counter in device memory (*step_d counts completed updates and is incremented by
 * the call): the same launch sequence can be captured in a CUDA graph and replayed. */
int stafb_adam_step_dev(stafb_ctx* ctx, void* stream, void* theta_d, const void* grad_d, void* m_d, void* v_d, int n,
                        double lr, double beta1, double beta2, double eps, int* step_d, double grad_scale);

/* Data-parallel training on the GPUs of one node without a collective library between the backward pass and the
 * optimiser: what hvd.DistributedOptimizer + Adam do in the reference (STAF/staf_train.py:484-487: average the
 * gradients over the ranks, then update) as ONE kernel per rank and step over NVLink peer memory.
 *   stafb_peer_create   allocates this rank's block: two gradient buffers (parity 0 / 1) and two receive areas
 *                       (one 8-byte word per source rank and element: the element's bits and its step number);
 *   stafb_peer_handle   writes the 64-byte CUDA IPC handle of that block (exchange them between the ranks by any
 *                       host-side means: torch.distributed.all_gather_object, MPI ...);
 *   stafb_peer_connect  maps the other ranks' blocks (handles[world][64], own entry ignored);
 *   stafb_peer_grad     device pointer of a gradient buffer: pass it as grad_d to stafb_train_step*;
 *   stafb_allreduce_adam  stores this rank's gradient, tagged with the step, into every peer's receive area (one
 *                       NVLink trip: value and tag travel in one word, no flag and no fence), waits until all
 *                       peers' elements of this step have arrived (bounded: about two seconds; then the launch as
 *                       a whole records STAFB_ERR_PEER_TIMEOUT and leaves theta, the moments and the step counter
 *                       untouched - one decision per launch, never a partial update), sums the gradients of
 *                       `parity` in rank order - bit-identical on every rank -, divides by the world size and
 *                       applies Adam (same formula and device step counter as stafb_adam_step_dev).  After a
 *                       timeout the ranks may hold different parameters (a late rank still finds the data of the
 *                       ranks that gave up): read stafb_peer_status on the host at regular points, re-broadcast
 *                       theta, the moments and the step count, and do not use this exchange again before
 *                       step numbers beyond those already published are reached (train.py continues with an
 *                       all-reduce).
 * Consecutive steps must alternate the parity; every rank must make the same calls in the same order.  The
 * blocks of the kernel wait for each other, so its grid must be resident as a whole: at most 8 x 256 parameters
 * per SM (STAFB_ERR_CAPACITY beyond).  Before stafb_peer_destroy all ranks must have finished their last step (a
 * host-side barrier). */
typedef struct stafb_peer stafb_peer;
int stafb_peer_create(stafb_ctx* ctx, int rank, int world, int n_params, stafb_peer** out);
int stafb_peer_handle(stafb_peer* p, void* handle64_out);
int stafb_peer_connect(stafb_peer* p, const void* handles);
/* ranks inside one process connect through their handles (all[world], own entry ignored), without IPC */
int stafb_peer_connect_local(stafb_peer* p, stafb_peer* const* all);
/* the two halves of stafb_allreduce_adam as separate launches (phase 1: store to the peers, 2: wait and update,
 * 3: both), for emulating several ranks on ONE GPU, where the ranks' kernels run one after the other and must
 * never wait for each other: every rank's phase 1 first, then every rank's phase 2 */
int stafb_allreduce_adam_phase(stafb_ctx* ctx, stafb_peer* p, void* stream, int parity, void* theta_d, void* m_d,
                               void* v_d, double lr, double beta1, double beta2, double eps, int* step_d, int phase);
/* bound of the wait for the peers' elements, in milliseconds of SM clock (default: about two seconds, or the
 * environment variable STAFB_PEER_WAIT_MS read by stafb_peer_create; 0 = give up at the first look) */
int stafb_peer_set_wait_ms(stafb_peer* p, long long ms);
void* stafb_peer_grad(stafb_peer* p, int parity);
int stafb_peer_status(stafb_peer* p);
void stafb_peer_destroy(stafb_peer* p);
int stafb_allreduce_adam(stafb_ctx* ctx, stafb_peer* p, void* stream, int parity, void* theta_d, void* m_d, void* v_d,
                         double lr, double beta1, double beta2, double eps, int* step_d);

/* The MLP head alone on caller-supplied fingerprints (what libstaf/include/staf_mlp.h:10-15 of the reference
 * defines for its pluggable MLP): energy_d[1] = 0.5 * sum of the atomic energies, dE_daf_d = d(sum of the atomic
 * energies)/dAF.  af_d and dE_daf_d: [N][Fmax] rows in the model's atom order (species-sorted; a species with fewer
 * fingerprints than Fmax leaves the tail of its rows unused).  One frame of the model's current atom counts. */
int stafb_mlp_eval(stafb_ctx* ctx, stafb_model* m, void* stream, const void* af_d, const void* theta_d,
                   const void* emb_d, void* energy_d, void* dE_daf_d);

/* Halo exchange of a slab decomposition over NVLink peer memory, for the ranks (one per GPU) of one node.  No
 * reference counterpart as a function: it is what LAMMPS' forward and reverse communication do around
 * PairSTAF::compute (lammps/USER-STAF/pair_staf.cpp:129-145 ghost atoms as neighbours, :250 forces on ghosts, summed
 * onto their owners by reverse_comm) without a message library on the path of an evaluation.  The periodic box is
 * cut into `world` slabs along one axis; rank r exchanges with lo = r-1 and hi = r+1 (mod world).  Each rank owns
 * one block that its peers map: its atom array (owned atoms | ghosts from lo | ghosts from hi; the neighbours store
 * their face atoms straight into the ghost regions), a receive area for the forces on the atoms it sent, per-rank
 * energies and flag words that carry the number of the evaluation.
 *   stafb_halo_create       allocates the block for at most cap_atoms atoms (owned + ghosts) and cap_face atoms per
 *                           face; every rank must pass the same two numbers (the peers address the block by them);
 *   stafb_halo_handle / _connect / _connect_local   as for stafb_peer_*;
 *   stafb_halo_positions    device pointer of the atom array [cap_atoms][3]: the caller keeps the owned positions in
 *                           its first n_own rows and passes it as positions_d to stafb_energy_force_domain;
 *   stafb_halo_forces       a [cap_atoms][3] array of the same type for that call's forces (convenience);
 *   stafb_halo_set_plan     which atoms leave through each face (indices among the owned atoms, device int32,
 *                           copied), how many ghosts arrive from each side, and where this rank's face atoms start
 *                           in the neighbour's array: dst_off_lo = first row of "ghosts from hi" in lo's array,
 *                           dst_off_hi = first row of "ghosts from lo" in hi's.  The ranks agree on these numbers
 *                           by any host-side means whenever the ghost sets are re-chosen.  All ranks must have
 *                           finished their evaluations under the old plan (a host-side barrier) before any sets
 *                           a new one;
 *   stafb_halo_plan_select / _layout / _done / _finish   the same agreement made on the device, for ranks that
 *                           cut the box into equal slabs along `axis` (0..2; box length L there): select picks the
 *                           owned atoms within `reach` (cutoff + skin) of this slab's faces, in index order, and
 *                           mails their number and species (types_d: int32 per owned atom) to the neighbours;
 *                           layout fills type_all_d[cap_atoms] (owned | from lo | from hi) and tells the
 *                           neighbours where their face atoms start; done waits for those answers; finish waits
 *                           for these three launches - the only host synchronisation -, puts the plan in force
 *                           and returns n_from_lo, n_from_hi, n_send_lo, n_send_hi.  No barrier between the ranks
 *                           is needed (a neighbour stores by the new offsets only after its own collect of the
 *                           evaluation before).  The new plan may be prepared one evaluation early: select, layout
 *                           (into a type_all array other than the one in use), done, then the push ... collect of
 *                           one more evaluation under the old plan, then finish - the host then never waits for
 *                           an idle GPU;
 *   one evaluation =  stafb_halo_push_positions; stafb_halo_wait_positions; stafb_energy_force_domain (energy_d =
 *                           the owned atoms' share, force_d for owned and ghost atoms); stafb_halo_return_forces
 *                           (ghost forces to their owners' ranks, this rank's energy to every rank);
 *                           stafb_halo_collect (adds the returned forces onto force_d's owned rows, writes the sum
 *                           of the ranks' energies, taken in rank order and so identical on every rank, to
 *                           energy_out_d, and advances the evaluation counter).  All five are asynchronous on
 *                           `stream` and read the evaluation number on the device, so the sequence may be captured
 *                           in a CUDA graph once per plan and replayed.
 * Every wait is bounded (about two seconds, STAFB_PEER_WAIT_MS or stafb_halo_set_wait_ms); after a miss
 * stafb_halo_status returns STAFB_ERR_PEER_TIMEOUT, the collect leaves the counter where it was and the results of
 * that evaluation are not valid.  Kernels of different ranks wait for each other: ranks that share ONE GPU (tests)
 * must issue all pushes before any wait, all returns before any collect, and each plan launch for all ranks
 * before the next. */
typedef struct stafb_halo stafb_halo;
int stafb_halo_create(stafb_ctx* ctx, int rank, int world, int cap_atoms, int cap_face, stafb_halo** out);
int stafb_halo_handle(stafb_halo* h, void* handle64_out);
int stafb_halo_connect(stafb_halo* h, const void* handles);
int stafb_halo_connect_local(stafb_halo* h, stafb_halo* const* all);
void* stafb_halo_positions(stafb_halo* h);
void* stafb_halo_forces(stafb_halo* h);
int stafb_halo_set_wait_ms(stafb_halo* h, long long ms);
int stafb_halo_set_plan(stafb_halo* h, void* stream, int n_own, int n_from_lo, int n_from_hi,
                        const int* send_lo_idx_d, int n_send_lo, int dst_off_lo, const int* send_hi_idx_d,
                        int n_send_hi, int dst_off_hi);
int stafb_halo_plan_select(stafb_halo* h, void* stream, int n_own, const int* types_d, int axis, double L,
                           double reach);
int stafb_halo_plan_layout(stafb_halo* h, void* stream, int* type_all_d);
int stafb_halo_plan_done(stafb_halo* h, void* stream);
int stafb_halo_plan_finish(stafb_halo* h, void* stream, int* counts_out4);
int stafb_halo_push_positions(stafb_halo* h, void* stream);
int stafb_halo_wait_positions(stafb_halo* h, void* stream);
int stafb_halo_return_forces(stafb_halo* h, void* stream, const void* force_d, const void* energy_d);
int stafb_halo_collect(stafb_halo* h, void* stream, void* force_d, void* energy_out_d);
int stafb_halo_status(stafb_halo* h);
void stafb_halo_destroy(stafb_halo* h);

/* Same as stafb_train_step but positions, boxer and labels are HOST buffers and losses is a
 * host double[4]: copies in, runs, copies the losses back and synchronises the stream. */
int stafb_train_step_host(stafb_ctx* ctx, stafb_model* m, void* stream, const void* positions_h, const void* boxer_h,
                          int nf, const void* theta_d, const void* emb_d, const void* e_label_h,
                          const void* f_label_h, double pe, double pf, double pb, double alpha_bound, int loss_kind,
                          double* losses_h, void* grad_d);

/* stafb_train_step_host split in two so that consecutive steps overlap: _begin stages the host inputs in the
 * slot's pinned block and enqueues the step on `stream` (the kernels read that block directly over PCIe and
 * write the losses and the status word straight into pinned memory; from the third call with the same
 * arguments on, the step is two replayed CUDA graphs: the neighbour rows on a stream of the model's own, where
 * they overlap the previous step, and the rest on `stream`) and returns at once; _end waits for that slot's step, writes losses_h[4] and returns the step's status
 * (STAFB_OK, STAFB_ERR_RADIAL_OVERFLOW, ...).  slot is 0 or 1; a slot must be collected with _end before it is
 * begun again.  Typical loop (what STAF/staf_train.py:678-755 does with a prefetch thread and TensorFlow's
 * asynchronous executor): begin(k, slot k&1); adam(k); end(k-1, slot (k-1)&1). */
int stafb_train_step_host_begin(stafb_ctx* ctx, stafb_model* m, void* stream, const void* positions_h,
                                const void* boxer_h, int nf, const void* theta_d, const void* emb_d,
                                const void* e_label_h, const void* f_label_h, double pe, double pf, double pb,
                                double alpha_bound, int loss_kind, void* grad_d, int slot);
int stafb_train_step_host_end(stafb_ctx* ctx, stafb_model* m, int slot, double* losses_h);

/* The same pair for the energy + force + virial step (stafb_train_step_virial; full_train_e_f_v,
 * STAF/staf_models/staf_model.py:313-384): v_label_h [nf,9] host virial labels (copied to the device by one small
 * transfer, all other inputs are read in place); _end writes losses_h[5] = loss, loss_e, loss_bound, loss_f,
 * loss_v.  The two pairs share the slots: a slot begun with one pair is collected with the same pair. */
int stafb_train_step_virial_host_begin(stafb_ctx* ctx, stafb_model* m, void* stream, const void* positions_h,
                                       const void* boxer_h, int nf, const void* theta_d, const void* emb_d,
                                       const void* e_label_h, const void* f_label_h, const void* v_label_h,
                                       double pe, double pf, double pv, double pb, double alpha_bound,
                                       int loss_kind, void* grad_d, int slot);
int stafb_train_step_virial_host_end(stafb_ctx* ctx, stafb_model* m, int slot, double* losses_h);

/* ---- diagnostics ----------------------------------------------------------------------------
 * The entry points from here to the end of the header are measurement aids of this library (no reference
 * counterpart, not part of the operator surface): phase timers, a measured FMA peak, a launch counter. */

/* Per-phase device timing of the fused calls, with CUDA events on the launching stream.  Phases, in order, of a
 * training evaluation: descriptors, af_fwd, mlp_fwd, force, force_grad, loss, mlp_bwd; of an inference
 * evaluation: descriptors, af_fwd, mlp_fwd, force, loss.  stafb_get_phase_times waits for the last event,
 * writes up to cap durations in milliseconds and returns how many.  Not for use while the stream is being
 * captured. */
int stafb_set_phase_timing(stafb_ctx* ctx, int on);
int stafb_get_phase_times(stafb_ctx* ctx, float* ms, int cap);

/* Measured FMA throughput of the current device in TFLOP/s (dtype STAFB_F32 or STAFB_F64): a register-resident
 * loop of independent fused multiply-adds on every SM, best of three runs, timed with CUDA events on `stream`.
 * The denominator for FP32 / FP64 pipe-utilisation figures (there is no reference counterpart). */
int stafb_measure_fma_peak(int dtype, void* stream, double* tflops_out);

/* number of kernels the last fused call launched (for accounting) */
int stafb_last_launch_count(const stafb_ctx* ctx);

#ifdef __cplusplus
}
#endif
#endif /* STAFB_H */
