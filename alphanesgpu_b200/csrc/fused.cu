// Fused energy/force/training path: descriptors never leave the chip.
//
// The operator path (ops.cu) has to honour the reference's tensor contract, which pushes
// ~110 KB per atom of angular descriptors (angdescr, intmap3b, der3b) through HBM.  Here the
// neighbour kernel leaves one compact record per atom (unit vectors, cutoffs, radial descriptors and
// their derivatives, neighbour ids, grouped by species: ~2 KB, common.cuh) and every sweep (sweep.cuh)
// rebuilds the triplet geometry in registers from the record staged in shared memory.
//
// This file: the evaluation's housekeeping kernel, the loss, Adam, the model handle and the launch
// sequences behind the fused entry points of include/stafb.h.  Math: STAF/staf_models/staf_model.py:168-258.
#include <math.h>
#include <stdlib.h>
#include <string.h>
#include <type_traits>
#include "common.cuh"

namespace stafb {

constexpr int ML_THREADS = 256;

struct ModelDev {
  int nt, C, N, ncls;
  int tipos[STAFB_MAX_TYPES], shift[STAFB_MAX_TYPES + 1], Fr[STAFB_MAX_TYPES], Fa[STAFB_MAX_TYPES];
  int off_a2[STAFB_MAX_TYPES], off_a3[STAFB_MAX_TYPES], off_mu[STAFB_MAX_TYPES], off_w[STAFB_MAX_TYPES];
  int off_emb[STAFB_MAX_TYPES];
  int n_dense, width[STAFB_MAX_DENSE];
  int Fmax, Frmax, Famax, Hsum, maxw;
  __host__ __device__ int in_of(int t, int l) const { return l == 0 ? Fr[t] + Fa[t] : width[l - 1]; }
  __host__ __device__ int w_off(int t, int l) const {
    int s = 0;
    for (int k = 0; k < l; k++) s += in_of(t, k) * width[k] + width[k];
    return s;
  }
  __host__ __device__ int h_off(int l) const {  // offset of the output of Dense l in the activation row
    int s = 0;
    for (int k = 0; k < l; k++) s += width[k];
    return s;
  }
  __host__ __device__ int type_of(int id) const {
    int t = 0;
    while (t < nt - 1 && id >= shift[t + 1]) t++;
    return t;
  }
};

// species-major enumeration: block -> (species t, index q0 of its first atom among the nf*tipos[t]
// atoms of that species); W atoms per block, blocks never mix species
__device__ __forceinline__ void locate_block(const ModelDev& md, int nf, int W, int& t, int& q0) {
  int blk = blockIdx.x;
  t = 0;
  while (t < md.nt - 1) {
    const int nb = (nf * md.tipos[t] + W - 1) / W;
    if (blk < nb) break;
    blk -= nb;
    t++;
  }
  q0 = blk * W;
}

__device__ __forceinline__ bool locate_atom(const ModelDev& md, int nf, int W, int slot, int& t, int& b, int& i) {
  int q0;
  locate_block(md, nf, W, t, q0);
  const int q = q0 + slot;
  if (q >= nf * md.tipos[t]) return false;
  b = q / md.tipos[t];
  i = md.shift[t] + (q - b * md.tipos[t]);
  return true;
}

static inline int species_blocks(const ModelDev& md, int nf, int W) {
  int s = 0;
  for (int t = 0; t < md.nt; t++) s += (nf * md.tipos[t] + W - 1) / W;
  return s;
}

#include "sweep.cuh"

// ---------------------------------------------------------------------------- MLP head
#include "mlp.cuh"
#include "mlp_mma.cuh"

// ---------------------------------------------------------------------------- energy, loss
template <class T>
__device__ __forceinline__ T huber(T e) { T a = r_abs(e); return a <= T(1) ? T(0.5) * e * e : a - T(0.5); }
template <class T>
__device__ __forceinline__ T huber_d(T e) { return e > T(1) ? T(1) : (e < T(-1) ? T(-1) : e); }

// Start-of-evaluation housekeeping in one launch: zero-fills up to three buffers (sizes in bytes, multiples of
// 4) and writes the packed, padded copy of the Dense layers that the MLP kernels stage (layout: mlp.cuh).
// It also packs the per-species parameter blocks of the sweeps (sweep.cuh): one warp per (species, class), and
// copies the force labels of a training evaluation into device scratch.
template <class T>
__global__ void k_prep(ModelDev md, const T* __restrict__ theta, const T* __restrict__ emb, T* __restrict__ wpack,
                       int wstride, unsigned char* __restrict__ spar, int spar_stride, SparLayout sl, void* a,
                       size_t na, void* b, size_t nb, void* c, size_t nc, const T* __restrict__ flab_src,
                       T* __restrict__ flab_dst, size_t nflab, T* __restrict__ wm, int wm_stride) {
  chain_wait();
  const size_t tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x, st = (size_t)gridDim.x * blockDim.x;
  // force labels into device scratch: the backward sweep gathers them per neighbour, and the caller's copy may
  // be mapped host memory (the host-buffer entry points), which is to be read exactly once
  for (size_t q = tid; q < nflab; q += st) flab_dst[q] = flab_src[q];
  {
    const int gw = (int)(tid >> 5), lane = threadIdx.x & 31;
    if (gw < md.nt * md.ncls) {
      const int t = gw / md.ncls, s = gw - t * md.ncls;
      spar_fill_class<T>(md, sl, spar + (size_t)t * spar_stride, t, s, theta, emb, lane);
    }
    for (int t = 0; t < md.nt; t++)
      for (size_t idx = tid; idx < (size_t)md.nt * md.Fr[t]; idx += st)
        spar_fill_radial<T>(md, sl, spar + (size_t)t * spar_stride, t, theta, emb, (int)idx);
  }
  for (size_t q = tid; q < na / 4; q += st) reinterpret_cast<int*>(a)[q] = 0;
  for (size_t q = tid; q < nb / 4; q += st) reinterpret_cast<int*>(b)[q] = 0;
  for (size_t q = tid; q < nc / 4; q += st) reinterpret_cast<int*>(c)[q] = 0;
  // one pass over all packed words: every thread's loads are independent, so the kernel costs one memory round trip
  for (size_t q = tid; q < (size_t)md.nt * wstride; q += st) {
    const int t = (int)(q / wstride);
    int r = (int)(q - (size_t)t * wstride), l = 0, woff = 0;
    while (l < md.n_dense && r >= ml_layer_words(md.in_of(t, l), md.width[l])) {
      r -= ml_layer_words(md.in_of(t, l), md.width[l]);
      woff += md.in_of(t, l) * md.width[l] + md.width[l];
      l++;
    }
    T v = T(0);
    if (l < md.n_dense) {
      const int out = md.width[l], ld = ml_ld(out);
      const int i = r / ld, j = r - i * ld;
      if (j < out) v = theta[md.off_w[t] + woff + i * out + j];  // row `in` is the bias
    }
    wpack[q] = v;
  }
  // the same layers split and ordered by MMA fragment for the tensor-core MLP kernels (mlp_mma.cuh; fp32 only)
  if constexpr (std::is_same<T, float>::value) {
    if (wm) {
      for (size_t q = tid; q < (size_t)md.nt * wm_stride; q += st) {
        const int t = (int)(q / wm_stride);
        int r = (int)(q - (size_t)t * wm_stride), l = 0;
        while (l < md.n_dense && r >= mm_layer_words(md.in_of(t, l), md.width[l])) {
          r -= mm_layer_words(md.in_of(t, l), md.width[l]);
          l++;
        }
        wm[q] = l < md.n_dense ? mm_pack_value(theta + md.off_w[t] + md.w_off(t, l), md.in_of(t, l), md.width[l], r)
                               : 0.0f;
      }
    }
  }
}

constexpr int LOSS_EB_MAX = 32;  // blocks that share the energy sum of one frame

// Losses of an evaluation in one launch.  Blocks [0,nf): frame energy E_b = 0.5*mean_i e_i (or 0.5*sum), energy
// loss and the cotangent on the atomic energies.  Blocks [nf, nf+fb): force loss (the backward sweep forms dL/dF
// itself, huber_d below is shared with it).  Last block: bound loss sum(alpha*[alpha>bound]) over alpha2b and
// alpha3b (Keras ReLU(threshold): staf_models/staf_model.py:60-62,215-219) and its gradient.  The block that
// finishes last adds up the total.  losses = {loss, loss_e, loss_bound, loss_f, done-counter}.
// In a training evaluation the kernel is launched AFTER the backward sweep of the forces, which does not need
// it: everything it reads (forces, atomic energies, theta) is at least two kernels old, so every block does its
// loads, arithmetic and reductions under the sweep's tail and waits for the chain only before its first global
// write.  In an inference evaluation it directly follows the force sweep; only the virial needs that one.
template <class T>
__global__ void __launch_bounds__(256)
    k_loss(ModelDev md, int nf, int eb, int fb, int per_atom, int train, const T* __restrict__ e_atom, T* __restrict__ energy,
           const T* __restrict__ e_label, const T* __restrict__ force, const T* __restrict__ f_label,
           const T* __restrict__ theta, T pe, T pf, T pb, T bound, int loss_kind, T* __restrict__ ebar,
           T* __restrict__ grad, double* __restrict__ losses, int* status, int* status_main,
           const double* __restrict__ vacc, T* __restrict__ virial_out, double* __restrict__ mirror,
           double* __restrict__ epart, unsigned* __restrict__ ecount, const T* __restrict__ v_label, T pv) {
  __shared__ double red[9];
  __shared__ int last_s;
  const int N = md.N;
  int blk = blockIdx.x;
  const bool needs_pred = (blk < nf * eb && virial_out);
  if (needs_pred) chain_wait();
  if (blk < nf * eb) {
    double Eb = 0.0;
    T le = T(0), de = T(0);
    // sum of the frame's atomic energies (the MLP kernel is at least two kernels back).  A large frame is summed
    // by eb blocks: each leaves its part, the one that arrives last adds the parts in their fixed order (the
    // result does not depend on which block that is) and finishes the frame.
    const int part = blk % eb;
    blk /= eb;
    const int per = (N + eb - 1) / eb, q1 = min(N, (part + 1) * per);
    double s = 0.0;
    for (int q = part * per + threadIdx.x; q < q1; q += blockDim.x) s += (double)e_atom[(size_t)blk * N + q];
    s = block_sum<double, 8>(s, red);
    if (eb > 1) {
      if (!needs_pred) chain_wait();
      unsigned* count = ecount + blk;
      if (threadIdx.x == 0) {
        epart[(size_t)blk * eb + part] = s;
        __threadfence();
        last_s = atomicAdd(count, 1u) == (unsigned)(eb - 1);
      }
      __syncthreads();
      if (!last_s) return;  // only inference evaluations use more than one block per frame
      if (threadIdx.x == 0) {
        __threadfence();
        s = 0.0;
        for (int k = 0; k < eb; k++) s += __ldcg(epart + (size_t)blk * eb + k);
        *count = 0u;
      }
    }
    if (threadIdx.x == 0) {
      Eb = per_atom ? 0.5 * s / N : 0.5 * s;
      if (train) {
        const T e = (T)Eb - e_label[blk];
        le = loss_kind == 0 ? huber(e) : e * e;
        de = loss_kind == 0 ? huber_d(e) : T(2) * e;
      }
    }
    if (!needs_pred && eb == 1) chain_wait();
    const double wv = ((virial_out || v_label) && threadIdx.x < 9) ? vir_total(vacc, blk, threadIdx.x) : 0.0;
    if (virial_out && threadIdx.x < 9) virial_out[blk * 9 + threadIdx.x] = (T)wv;
    if (v_label && threadIdx.x < 9) {
      // virial term of the loss (staf_model.py:358-365): mean over [nf, 9]; its cotangent is formed by the
      // backward sweep of the forces itself.  losses[5] (losses[4] is the done-counter).
      const T e = (T)wv - v_label[blk * 9 + threadIdx.x];
      atomicAdd(losses + 5, (double)(loss_kind == 0 ? huber(e) : e * e) / (9.0 * nf));
    }
    if (threadIdx.x == 0) {
      if (!isfinite(Eb)) set_status(status, STAFB_ERR_NONFINITE);
      if (energy) energy[blk] = (T)Eb;
      if (train) {
        atomicAdd(losses + 1, (double)le / nf);
        ebar[blk] = pe * de / T(nf) * T(0.5) / (per_atom ? T(N) : T(1));
      }
    }
  } else if (blk < nf * eb + fb) {
    const size_t n = (size_t)nf * 3 * N;
    double s = 0.0;
    for (size_t q = (size_t)(blk - nf * eb) * blockDim.x + threadIdx.x; q < n; q += (size_t)fb * blockDim.x) {
      const T e = force[q] - f_label[q];
      s += (double)(loss_kind == 0 ? huber(e) : e * e);
    }
    s = block_sum<double, 8>(s, red);
    chain_wait();
    if (threadIdx.x == 0) atomicAdd(losses + 3, s / (double)n);
  } else {
    // bound term: the sum under the predecessor's tail, the gradient contributions after the wait
    double s = 0.0;
    for (int t = 0; t < md.nt; t++) {
      const int n2 = md.nt * md.Fr[t], n3 = md.C * 3 * md.Fa[t];
      for (int q = threadIdx.x; q < n2 + n3; q += blockDim.x) {
        const T x = theta[q < n2 ? md.off_a2[t] + q : md.off_a3[t] + (q - n2)];
        if (x > bound) s += (double)x;
      }
    }
    s = block_sum<double, 8>(s, red);
    chain_wait();
    for (int t = 0; t < md.nt; t++) {
      const int n2 = md.nt * md.Fr[t], n3 = md.C * 3 * md.Fa[t];
      for (int q = threadIdx.x; q < n2 + n3; q += blockDim.x) {
        const int idx = q < n2 ? md.off_a2[t] + q : md.off_a3[t] + (q - n2);
        if (theta[idx] > bound) atomicAdd(grad + idx, pb);
      }
    }
    if (threadIdx.x == 0) atomicAdd(losses + 2, s);
  }
  if (train && threadIdx.x == 0) {
    __threadfence();
    const unsigned done = atomicAdd(reinterpret_cast<unsigned*>(losses + 4), 1u);
    if (done == gridDim.x - 1) {
      __threadfence();
      const double le = atomicAdd(losses + 1, 0.0), lb = atomicAdd(losses + 2, 0.0), lf = atomicAdd(losses + 3, 0.0);
      const double lv = v_label ? atomicAdd(losses + 5, 0.0) : 0.0;
      const double tot = (double)pe * le + (double)pb * lb + (double)pf * lf + (double)pv * lv;
      losses[0] = tot;
      if (mirror) {
        // results straight into the caller's mapped host memory: 4 losses, the status word (read and cleared),
        // the virial loss
        mirror[0] = tot; mirror[1] = le; mirror[2] = lb; mirror[3] = lf; mirror[5] = lv;
        reinterpret_cast<int*>(mirror + 4)[0] = atomicExch(status, 0);
        __threadfence_system();
      } else if (status_main != status) {
        // prefetched neighbour rows report into their own word: hand it over to the context's
        const int v = atomicExch(status, 0);
        if (v) set_status(status_main, v);
      }
    }
  }
}

template <class T>
__global__ void k_adam(int n, T* __restrict__ theta, const T* __restrict__ grad, T* __restrict__ m,
                       T* __restrict__ v, T lr_t, T b1, T b2, T eps, T gscale) {  chain_wait();

  const int q = blockIdx.x * blockDim.x + threadIdx.x;
  if (q >= n) return;
  const T g = grad[q] * gscale;
  const T mm = b1 * m[q] + (T(1) - b1) * g;
  const T vv = b2 * v[q] + (T(1) - b2) * g * g;
  m[q] = mm;
  v[q] = vv;
  theta[q] -= lr_t * mm / (r_sqrt(vv) + eps);
}

// Adam with the step count kept on the device, so that a captured CUDA graph can be replayed.
// Every thread reads the counter; the block that finishes last increments it.
template <class T>
__global__ void k_adam_dev(int n, T* __restrict__ theta, const T* __restrict__ grad, T* __restrict__ m,
                           T* __restrict__ v, double lr, double b1, double b2, T eps, T gscale,
                           int* __restrict__ step_d /*[2]: step, blocks done*/) {  chain_wait();

  const int q = blockIdx.x * blockDim.x + threadIdx.x;
  const int step = *reinterpret_cast<volatile int*>(step_d) + 1;
  if (q < n) {
    const T lr_t = (T)(lr * sqrt(1.0 - pow(b2, (double)step)) / (1.0 - pow(b1, (double)step)));
    const T g = grad[q] * gscale;
    const T mm = (T)b1 * m[q] + (T(1) - (T)b1) * g;
    const T vv = (T)b2 * v[q] + (T(1) - (T)b2) * g * g;
    m[q] = mm;
    v[q] = vv;
    theta[q] -= lr_t * mm / (r_sqrt(vv) + eps);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(step_d + 1, 1) == (int)gridDim.x - 1) {
      step_d[1] = 0;
      __threadfence();
      atomicAdd(step_d, 1);
    }
  }
}

}  // namespace stafb

using namespace stafb;

struct stafb_model {
  stafb_ctx* ctx;
  ModelDev md;
  int n_params, n_emb;
  int blk_size[STAFB_MAX_TYPES];
  size_t es;
  int cap_atoms;  // atoms per frame the scratch was sized for
  int aw;   // atoms per warp of the MLP kernels (4, 2 or 1; a block of eight warps owns 8*aw atoms)
  int stage;  // Dense layers in shared memory: 2 all at kernel start, 1 one at a time, 0 none
  size_t mlp_fwd_smem, mlp_bwd_smem;
  // scratch for max_batch frames
  void *rows, *af, *nd, *acts, *e_atom, *force, *flab, *ebar, *gradnet, *gaf, *energy, *vrow;
  int row_stride;      // bytes per neighbour record (common.cuh)
  unsigned char* spar;  // per-species parameter blocks of the sweeps, rewritten by k_prep at every evaluation
  SparLayout sl;
  void* wpack;  // packed, padded Dense layers of every species (k_prep), wstride elements per species
  int wstride;
  int nv;  // row length of vrow: nt*Frmax + C*3*Famax
  // tensor-core MLP kernels (fp32): on/off, warps per block (16 atoms), the fragment-ordered pack and its
  // per-species stride, dynamic shared memory of the two kernels
  int mma, mma_nw, mma_stage, wm_stride;
  void* wm;
  size_t mma_fwd_smem, mma_bwd_smem;
  double* epart;     // partial energy sums of k_loss: [nf][eb]; from [max_batch][LOSS_EB_MAX] on: one arrival counter per frame
  double* losses_d;  // [0..4] the four losses + the done-counter of k_loss; [8 + b] sum of the atomic energies of
                     // frame b (accumulated by the MLP kernel); from [8 + max_batch] on the virial accumulators [b][9][VIR_SLOTS]
  // staging for the *_host entry points
  // two pipelined slots for stafb_train_step_host_begin/_end: pinned input block (pos | f_label | box | e_label),
  // pinned results (4 losses + status) and the event that marks the slot's step complete
  char* slot_in_h[3];  // slots 0, 1: the pipelined calls; slot 2: the synchronous stafb_train_step_host
  double* slot_out_h[3];
  cudaEvent_t slot_done[3];
  int slot_busy[3];
  // per slot: the captured graph of (copy in, step, copy out) and the call signature it was captured for
  struct SlotKey {
    int nf, loss_kind;
    const void *theta, *emb, *grad, *stream;
    double pe, pf, pb, bound, pv;
    int with_v;
  } slot_key[3];
  double* mirror_next;  // mapped host memory the next training evaluation's k_loss writes its results to
  void* vlab_d;         // device copy of the virial labels of a host-buffer step [max_batch][9]
  int slot_state[3];  // 0: nothing yet, 1: signature seen once (ran eagerly), 2: graph instantiated, -1: capture failed
  cudaGraphExec_t slot_exec[3];
  // Two more sets of neighbour rows (a context of their own for the search scratch + the compact rows), so that
  // the geometry of the NEXT step, which depends on no trainable parameter, can be built on another stream while
  // this step's sweeps still read theirs.  Allocated on first use.
  struct NlSet {
    stafb_ctx* ctx;
    void* rows;
    cudaEvent_t ready;
    int nf;  // frames the set currently describes (0: nothing)
  } nl[2];
  cudaStream_t side;  // stream of the prefetches issued by stafb_train_step_host_begin
  cudaGraphExec_t nl_exec[2];
  size_t smem_limit;
};

// words of shared memory the staged Dense layers need: stage 1 = the largest (in + 1) x row stride over the
// layers, stage 2 = all layers of one species back to back
static size_t mlp_stage_words(const ModelDev& d, int stage) {
  size_t best = 0;
  for (int t = 0; t < d.nt; t++) {
    size_t sum = 0;
    for (int l = 0; l < d.n_dense; l++) {
      const size_t wds = (size_t)(d.in_of(t, l) + 1) * ml_ld(d.width[l]);
      sum += wds;
      if (stage == 1) best = wds > best ? wds : best;
    }
    if (stage == 2) best = sum > best ? sum : best;
  }
  return stage ? best : 0;
}
static size_t mlp_smem_fwd(const ModelDev& d, size_t es, int aw, int stage) {
  return es * (ML_WARPS * ml_fwd_words(d.Fmax, d.Hsum, d.maxw, aw) + mlp_stage_words(d, stage));
}
static size_t mlp_smem_bwd(const ModelDev& d, size_t es, int aw, int stage) {
  return es * (ML_WARPS * ml_bwd_words(d.Fmax, d.Hsum, d.maxw, aw) + mlp_stage_words(d, stage));
}

extern "C" int stafb_model_create(stafb_ctx* c, const int* sd, stafb_model** out) {
  if (!c || !sd || !out) return STAFB_ERR_INVALID;
  stafb_model* m = (stafb_model*)calloc(1, sizeof(stafb_model));
  ModelDev& d = m->md;
  d.nt = sd[0];
  if (d.nt < 1 || d.nt > STAFB_MAX_TYPES) { free(m); return STAFB_ERR_INVALID; }
  d.C = d.nt * (d.nt + 1) / 2;
  d.ncls = d.C < 2 * d.nt - 1 ? d.C : 2 * d.nt - 1;
  d.n_dense = sd[13];
  if (d.n_dense < 1 || d.n_dense > STAFB_MAX_DENSE) { free(m); return STAFB_ERR_INVALID; }
  for (int l = 0; l < d.n_dense; l++) d.width[l] = sd[14 + l];
  if (d.width[d.n_dense - 1] != 1) { free(m); return STAFB_ERR_INVALID; }
  d.N = 0;
  d.Fmax = d.Frmax = d.Famax = 0;
  d.shift[0] = 0;
  int off = 0, eoff = 0;
  for (int t = 0; t < d.nt; t++) {
    d.tipos[t] = sd[1 + t];
    d.Fr[t] = sd[5 + t];
    d.Fa[t] = sd[9 + t];
    if (d.tipos[t] < 0 || d.Fr[t] < 0 || d.Fa[t] < 0 || d.Fa[t] > 255) { free(m); return STAFB_ERR_INVALID; }
    d.shift[t + 1] = d.shift[t] + d.tipos[t];
    d.N += d.tipos[t];
    const int F = d.Fr[t] + d.Fa[t];
    d.Fmax = F > d.Fmax ? F : d.Fmax;
    d.Frmax = d.Fr[t] > d.Frmax ? d.Fr[t] : d.Frmax;
    d.Famax = d.Fa[t] > d.Famax ? d.Fa[t] : d.Famax;
    d.off_a2[t] = off;
    d.off_a3[t] = d.off_a2[t] + d.nt * d.Fr[t];
    d.off_mu[t] = d.off_a3[t] + d.C * 3 * d.Fa[t];
    d.off_w[t] = d.off_mu[t] + F;
    int nw = 0, in = F;
    for (int l = 0; l < d.n_dense; l++) { nw += in * d.width[l] + d.width[l]; in = d.width[l]; }
    m->blk_size[t] = d.nt * d.Fr[t] + d.C * 3 * d.Fa[t] + F + nw;
    off += m->blk_size[t];
    d.off_emb[t] = eoff;
    eoff += d.nt * d.Fr[t] + d.C * d.Fa[t];
  }
  if (d.N > c->n_max) { free(m); return STAFB_ERR_CAPACITY; }
  d.Hsum = 0;
  d.maxw = d.Fmax;
  for (int l = 0; l < d.n_dense; l++) { d.Hsum += d.width[l]; d.maxw = d.width[l] > d.maxw ? d.width[l] : d.maxw; }
  m->n_params = off;
  m->n_emb = eoff;
  m->ctx = c;
  m->es = c->dtype == STAFB_F32 ? 4 : 8;
  int dev = 0, lim = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&lim, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
  m->smem_limit = (size_t)lim;
  m->aw = 0;
  int nsm = 148;
  cudaDeviceGetAttribute(&nsm, cudaDevAttrMultiProcessorCount, dev);
  // Atoms per warp of the MLP kernels and where the Dense layers live.  Wanted: many resident warps (4 atoms per
  // warp only if that still gives four blocks per SM, else 2: the kernels are latency-bound until the GPU is full,
  // and the backward kernel's slices at 4 atoms per warp leave room for one block per SM only) and all layers
  // staged in shared memory at kernel start
  // (2); what does not fit falls back to one layer at a time (1), then to fewer atoms per warp, then to reading
  // the weights from global memory (0).
  const size_t mlp_room = m->smem_limit - 1024;  // the backward kernel also holds a little static shared memory
  const int aw_pref = species_blocks(d, c->max_batch, ML_WARPS * 4) >= 4 * nsm ? 4 : 2;
  const int cand[7][2] = {{aw_pref, 2}, {aw_pref, 1}, {2, 1}, {1, 1}, {aw_pref, 0}, {2, 0}, {1, 0}};
  m->stage = 0;
  for (int k = 0; k < 7 && !m->aw; k++)
    if (mlp_smem_bwd(d, m->es, cand[k][0], cand[k][1]) <= mlp_room) { m->aw = cand[k][0]; m->stage = cand[k][1]; }
  if (getenv("STAFB_MLP_STAGE")) m->stage = atoi(getenv("STAFB_MLP_STAGE"));
  if (getenv("STAFB_MLP_AW")) m->aw = atoi(getenv("STAFB_MLP_AW"));
  if (m->aw != 1 && m->aw != 2 && m->aw != 4) { free(m); return STAFB_ERR_CAPACITY; }
  if (m->stage < 0 || m->stage > 2 || mlp_smem_bwd(d, m->es, m->aw, m->stage) > mlp_room) { free(m); return STAFB_ERR_CAPACITY; }
  m->mlp_fwd_smem = mlp_smem_fwd(d, m->es, m->aw, m->stage);
  m->mlp_bwd_smem = mlp_smem_bwd(d, m->es, m->aw, m->stage);
  // The tensor-core form of the MLP kernels (mlp_mma.cuh; fp32 only, one block per 16 atoms, its warps - 4;
  // STAFB_MLP_MMA_NW: 1, 2, 4, 8 - sharing the tiles) is the other arm, selected with STAFB_MLP_MMA=1: on B200
  // mma.sync.m16n8k8.tf32 issues at about one instruction per 30 cycles per SM, which leaves these kernels
  // 1.4-2x behind the FMA kernels at every size measured (768-atom frames at batch 4, 8, 16; a 24,576-atom box).
  m->mma = 0; m->wm = nullptr; m->wm_stride = 0;
  if (c->dtype == STAFB_F32 && d.width[d.n_dense - 1] == 1 && !getenv("STAFB_MLP_STAGE") &&
      getenv("STAFB_MLP_MMA") && atoi(getenv("STAFB_MLP_MMA")) == 1) {
    const size_t fw = 4 * mm_fwd_words(d), bw = 4 * mm_bwd_words(d);
    int nw = getenv("STAFB_MLP_MMA_NW") ? atoi(getenv("STAFB_MLP_MMA_NW")) : 4;
    if ((nw == 1 || nw == 2 || nw == 4 || nw == 8) && bw <= mlp_room && fw <= mlp_room) {
      m->mma = 1; m->mma_nw = nw; m->mma_stage = 0;
      m->mma_fwd_smem = fw; m->mma_bwd_smem = bw;
      m->wm_stride = (int)mm_pack_words(d);
    }
  }
  // scratch is sized for the context's atom capacity, so that stafb_model_set_counts can move atoms between
  // species (or change their number) without reallocating
  const size_t es = m->es, A = (size_t)c->max_batch * c->n_max, nr = c->nr;
  m->cap_atoms = c->n_max;
  const size_t mlp_blocks = A / (ML_WARPS * m->aw) + d.nt + 1;
  m->row_stride = row_stride_bytes((int)nr, (int)es);
  STAFB_CUDA_OK(cudaMalloc(&m->rows, A * (size_t)m->row_stride));
  STAFB_CUDA_OK(cudaMemset(m->rows, 0, A * (size_t)m->row_stride));
  m->sl = es == 4 ? spar_layout<float>(d) : spar_layout<double>(d);
  STAFB_CUDA_OK(cudaMalloc((void**)&m->spar, (size_t)d.nt * m->sl.total));
  STAFB_CUDA_OK(cudaMemset(m->spar, 0, (size_t)d.nt * m->sl.total));
  STAFB_CUDA_OK(cudaMalloc(&m->af, es * A * d.Fmax));
  STAFB_CUDA_OK(cudaMalloc(&m->nd, es * A * d.Fmax));
  STAFB_CUDA_OK(cudaMalloc(&m->gradnet, es * A * d.Fmax));
  STAFB_CUDA_OK(cudaMalloc(&m->gaf, es * A * d.Fmax));
  m->nv = d.nt * d.Frmax + d.C * 3 * d.Famax;
  STAFB_CUDA_OK(cudaMalloc(&m->vrow, es * A * (m->nv > 0 ? m->nv : 1)));
  {
    size_t acts_words = mlp_blocks * ML_WARPS * m->aw * d.Hsum;
    if (m->mma) {
      const size_t tiles = A / MM_ATOMS + (size_t)d.nt * c->max_batch + 1;
      const size_t w2 = tiles * MM_ATOMS * (size_t)mm_shape(d, 0).hoff[d.n_dense];
      acts_words = w2 > acts_words ? w2 : acts_words;
      STAFB_CUDA_OK(cudaMalloc(&m->wm, sizeof(float) * (size_t)d.nt * m->wm_stride));
    }
    STAFB_CUDA_OK(cudaMalloc(&m->acts, es * acts_words));
  }
  m->wstride = (int)mlp_stage_words(d, 2);
  STAFB_CUDA_OK(cudaMalloc(&m->wpack, es * (size_t)d.nt * m->wstride));
  STAFB_CUDA_OK(cudaMalloc(&m->e_atom, es * A));
  STAFB_CUDA_OK(cudaMalloc(&m->force, es * A * 3));
  STAFB_CUDA_OK(cudaMalloc(&m->flab, es * A * 3));  // device copy of the force labels (k_prep)
  STAFB_CUDA_OK(cudaMalloc(&m->ebar, es * c->max_batch));
  STAFB_CUDA_OK(cudaMalloc(&m->energy, es * c->max_batch));
  // 8 loss words, a counter per frame, the virial accumulators
  STAFB_CUDA_OK(cudaMalloc((void**)&m->losses_d, sizeof(double) * (8 + (1 + 9 * VIR_SLOTS) * (size_t)c->max_batch)));
  STAFB_CUDA_OK(cudaMalloc((void**)&m->epart, sizeof(double) * (size_t)c->max_batch * (LOSS_EB_MAX + 1)));
  STAFB_CUDA_OK(cudaMemset(m->epart, 0, sizeof(double) * (size_t)c->max_batch * (LOSS_EB_MAX + 1)));
  {
    const size_t blk = es * (A * 6 + (size_t)c->max_batch * 16 + 8);  // pos | f_label | box | e_label | v_label
    STAFB_CUDA_OK(cudaMalloc(&m->vlab_d, es * (size_t)c->max_batch * 9));
    for (int k = 0; k < 3; k++) {
      STAFB_CUDA_OK(cudaMallocHost((void**)&m->slot_in_h[k], blk));
      STAFB_CUDA_OK(cudaMallocHost((void**)&m->slot_out_h[k], sizeof(double) * 6));
      STAFB_CUDA_OK(cudaEventCreateWithFlags(&m->slot_done[k], cudaEventDisableTiming));
      m->slot_busy[k] = 0;
    }
  }
  *out = m;
  return STAFB_OK;
}

extern "C" void stafb_model_destroy(stafb_model* m) {
  if (!m) return;
  void* ptrs[] = {m->rows, m->spar, m->af, m->nd, m->gradnet, m->gaf, m->acts, m->e_atom, m->force,
                  m->flab, m->ebar, m->energy, m->losses_d, m->epart, m->vrow, m->wpack, m->wm, m->vlab_d};
  for (void* p : ptrs) cudaFree(p);
  for (int k = 0; k < 3; k++) {
    cudaFreeHost(m->slot_in_h[k]);
    cudaFreeHost(m->slot_out_h[k]);
    if (m->slot_done[k]) cudaEventDestroy(m->slot_done[k]);
    if (m->slot_exec[k]) cudaGraphExecDestroy(m->slot_exec[k]);
  }
  for (int k = 0; k < 2; k++) {
    if (m->nl_exec[k]) cudaGraphExecDestroy(m->nl_exec[k]);
    if (!m->nl[k].ctx) continue;
    cudaFree(m->nl[k].rows);
    cudaEventDestroy(m->nl[k].ready);
    stafb_destroy(m->nl[k].ctx);
  }
  if (m->side) cudaStreamDestroy(m->side);
  free(m);
}

extern "C" int stafb_model_set_counts(stafb_model* m, const int* tipos) {
  if (!m || !tipos) return STAFB_ERR_INVALID;
  ModelDev& d = m->md;
  int n = 0;
  for (int t = 0; t < d.nt; t++) {
    if (tipos[t] < 0) return STAFB_ERR_INVALID;
    n += tipos[t];
  }
  if (n <= 0) return STAFB_ERR_INVALID;
  if (n > m->cap_atoms) return STAFB_ERR_CAPACITY;
  d.shift[0] = 0;
  for (int t = 0; t < d.nt; t++) {
    d.tipos[t] = tipos[t];
    d.shift[t + 1] = d.shift[t] + tipos[t];
  }
  d.N = n;
  return STAFB_OK;
}

extern "C" int stafb_model_n_params(const stafb_model* m) { return m ? m->n_params : -1; }
extern "C" int stafb_model_n_emb(const stafb_model* m) { return m ? m->n_emb : -1; }
extern "C" void stafb_model_mlp_config(const stafb_model* m, int out4[4]) {
  out4[0] = m->stage; out4[1] = m->aw; out4[2] = (int)m->mlp_fwd_smem; out4[3] = (int)m->mlp_bwd_smem;
}

extern "C" void stafb_model_mlp_mma_config(const stafb_model* m, int out4[4]) {
  out4[0] = m->mma; out4[1] = m->mma ? m->mma_nw : 0; out4[2] = m->mma ? m->mma_stage : 0;
  out4[3] = m->mma ? (int)m->mma_bwd_smem : 0;
}
extern "C" void stafb_model_offsets(const stafb_model* m, int t, int out6[6]) {
  out6[0] = m->md.off_a2[t]; out6[1] = m->md.off_a3[t]; out6[2] = m->md.off_mu[t]; out6[3] = m->md.off_w[t];
  out6[4] = m->md.off_emb[t]; out6[5] = m->blk_size[t];
}

// cudaFuncSetAttribute applies to the device that is current when it is called, and one process may drive
// several GPUs (staf_load honours StafOptions.device_id; stafb_peer_connect_local exists for that use): the
// "already opted in" notes of the launchers below are therefore kept per device, as the reference keeps its
// per-device context map (STAF/src/descriptor_builder/reforce.cc:143-158).
constexpr int MAX_DEVICES = 64;
static inline int device_slot() {
  int d = 0;
  cudaGetDevice(&d);
  return (d >= 0 && d < MAX_DEVICES) ? d : 0;
}

// what a sweep launch needs besides the model: the records of this evaluation and the per-call buffers
template <class T>
struct SweepCall {
  const void* rows;
  int nf, nall;
  const T* chan_in;
  const T* force;  // force-backward sweep: the forces, their labels and the loss's scale (dL/dF is formed on the fly)
  const T* flab;
  T fscale;
  int loss_kind;
  T* out;
  T* grad;
  T* vout;
  double* vir;
  const double* vacc;  // force backward with a virial loss: the virials, their labels, the loss's scale
  const T* vlab;
  T vscale;
  int* status;
};

template <class T, int MODE>
static int launch_sweep(stafb_model* m, cudaStream_t s, const SweepCall<T>& call) {
  const ModelDev& d = m->md;
  const int nr = m->ctx->nr;
  const SweepSmem L = sweep_smem<T>(d, m->sl, nr, MODE);
  const size_t sm = (size_t)L.total;
  if (sm > m->smem_limit) return STAFB_ERR_CAPACITY;
  static bool attr_dev[MAX_DEVICES] = {false};  // per instantiation (T, MODE) and device
  bool& attr_done = attr_dev[device_slot()];
  if (sm > 48 * 1024 && !attr_done) {
    STAFB_CUDA_OK(cudaFuncSetAttribute(k_sweep<T, MODE, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       (int)m->smem_limit));
    if (MODE == MODE_FORCE)
      STAFB_CUDA_OK(cudaFuncSetAttribute(k_sweep<T, MODE, MODE == MODE_FORCE>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)m->smem_limit));
    attr_done = true;
  }
  SweepArgs<T> a;
  a.rows = static_cast<const unsigned char*>(call.rows);
  a.row_stride = m->row_stride;
  a.nr = nr; a.nf = call.nf; a.nall = call.nall;
  a.spar = m->spar;
  a.spar_stride = m->sl.total;
  a.sl = m->sl;
  a.chan_in = call.chan_in; a.force = call.force; a.flab = call.flab; a.fscale = call.fscale;
  a.loss_kind = call.loss_kind; a.out = call.out; a.grad = call.grad;
  a.vout = call.vout; a.nv = m->nv; a.vir = call.vir; a.status = call.status;
  a.vacc = call.vacc; a.vlab = call.vlab; a.vscale = call.vscale;
  const int blocks = call.nf * d.N;
  if (MODE == MODE_FORCE && call.vir)
    STAFB_CUDA_OK(launch_chained(k_sweep<T, MODE, MODE == MODE_FORCE>, blocks, 32, sm, s, d, a, L));
  else
    STAFB_CUDA_OK(launch_chained(k_sweep<T, MODE, false>, blocks, 32, sm, s, d, a, L));
  m->ctx->launches++;
  return STAFB_OK;
}

// where the neighbour kernels leave the records of a model's atoms
static RowSink row_sink(const stafb_model* m, void* rows, const int* tmap) {
  RowSink sk;
  memset(&sk, 0, sizeof(sk));
  sk.rows = rows;
  sk.stride = m->row_stride;
  sk.nt = m->md.nt;
  for (int t = 0; t <= m->md.nt; t++) sk.shift[t] = m->md.shift[t];
  sk.tmap = tmap;
  return sk;
}

template <class T, int AW, bool WG, bool WIDE>
static int launch_mlp_fwd_t(stafb_model* m, cudaStream_t s, int nf, const T* theta, const T* af, T* acts, T* e_atom,
                            T* nd) {
  static size_t attr_dev[MAX_DEVICES] = {0};  // largest dynamic shared-memory size opted in for, per device
  size_t& attr = attr_dev[device_slot()];
  if (m->mlp_fwd_smem > 48 * 1024 && m->mlp_fwd_smem > attr) {
    STAFB_CUDA_OK(cudaFuncSetAttribute(k_mlp_fwd<T, AW, WG, WIDE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       (int)m->mlp_fwd_smem));
    attr = m->mlp_fwd_smem;
  }
  STAFB_CUDA_OK(launch_chained(k_mlp_fwd<T, AW, WG, WIDE>, species_blocks(m->md, nf, ML_WARPS * AW), ML_THREADS,
                               m->mlp_fwd_smem, s, m->md, nf, theta, (const T*)m->wpack, m->wstride, af, acts, e_atom,
                               nd, m->stage, (int)mlp_stage_words(m->md, m->stage)));
  m->ctx->launches++;
  return STAFB_OK;
}

template <class T, int AW, bool WG, bool WIDE>
static int launch_mlp_bwd_t(stafb_model* m, cudaStream_t s, int nf, const T* theta, const T* af, const T* acts,
                            const T* ebar, const T* u, T* gaf, T* grad) {
  static size_t attr_dev[MAX_DEVICES] = {0};
  size_t& attr = attr_dev[device_slot()];
  const T* vrow = (const T*)m->vrow;
  if (m->mlp_bwd_smem > 48 * 1024 && m->mlp_bwd_smem > attr) {
    STAFB_CUDA_OK(cudaFuncSetAttribute(k_mlp_bwd<T, AW, WG, WIDE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       (int)m->mlp_bwd_smem));
    attr = m->mlp_bwd_smem;
  }
  STAFB_CUDA_OK(launch_chained(k_mlp_bwd<T, AW, WG, WIDE>, species_blocks(m->md, nf, ML_WARPS * AW), ML_THREADS,
                               m->mlp_bwd_smem, s, m->md, nf, theta, (const T*)m->wpack, m->wstride, af, acts, ebar, u,
                               vrow, m->nv, gaf, grad, m->stage, (int)mlp_stage_words(m->md, m->stage)));
  m->ctx->launches++;
  return STAFB_OK;
}

static int launch_mlp_fwd_mma(stafb_model* m, cudaStream_t s, int nf, const float* theta, const float* af, float* acts,
                              float* e_atom, float* nd) {
  static size_t attr_dev[MAX_DEVICES] = {0};
  size_t& attr = attr_dev[device_slot()];
  if (m->mma_fwd_smem > 48 * 1024 && m->mma_fwd_smem > attr) {
    STAFB_CUDA_OK(cudaFuncSetAttribute(k_mlp_fwd_mma, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       (int)m->mma_fwd_smem));
    attr = m->mma_fwd_smem;
  }
  STAFB_CUDA_OK(launch_chained(k_mlp_fwd_mma, species_blocks(m->md, nf, MM_ATOMS), 32 * m->mma_nw, m->mma_fwd_smem, s,
                               m->md, nf, theta, (const float*)m->wm, m->wm_stride, af, acts, e_atom, nd));
  m->ctx->launches++;
  return STAFB_OK;
}

static int launch_mlp_bwd_mma(stafb_model* m, cudaStream_t s, int nf, const float* theta, const float* af,
                              const float* acts, const float* ebar, const float* u, float* gaf, float* grad) {
  static size_t attr_dev[MAX_DEVICES] = {0};
  size_t& attr = attr_dev[device_slot()];
  if (m->mma_bwd_smem > 48 * 1024 && m->mma_bwd_smem > attr) {
    STAFB_CUDA_OK(cudaFuncSetAttribute(k_mlp_bwd_mma, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       (int)m->mma_bwd_smem));
    attr = m->mma_bwd_smem;
  }
  STAFB_CUDA_OK(launch_chained(k_mlp_bwd_mma, species_blocks(m->md, nf, MM_ATOMS), 32 * m->mma_nw, m->mma_bwd_smem, s,
                               m->md, nf, theta, (const float*)m->wm, m->wm_stride, af, acts, ebar, u,
                               (const float*)m->vrow, m->nv, gaf, grad));
  m->ctx->launches++;
  return STAFB_OK;
}

template <class T>
static int launch_mlp_fwd(stafb_model* m, cudaStream_t s, int nf, const T* theta, const T* af, T* acts, T* e_atom,
                          T* nd) {
  if constexpr (std::is_same<T, float>::value) {
    if (m->mma) return launch_mlp_fwd_mma(m, s, nf, theta, af, acts, e_atom, nd);
  }
  const bool wg = m->stage == 0, wide = m->md.maxw > 64;  // the dense products' form: see mlp.cuh
  switch (m->aw) {
    case 4: return wg ? (wide ? launch_mlp_fwd_t<T, 4, true, true>(m, s, nf, theta, af, acts, e_atom, nd) : launch_mlp_fwd_t<T, 4, true, false>(m, s, nf, theta, af, acts, e_atom, nd))
                      : (wide ? launch_mlp_fwd_t<T, 4, false, true>(m, s, nf, theta, af, acts, e_atom, nd) : launch_mlp_fwd_t<T, 4, false, false>(m, s, nf, theta, af, acts, e_atom, nd));
    case 2: return wg ? (wide ? launch_mlp_fwd_t<T, 2, true, true>(m, s, nf, theta, af, acts, e_atom, nd) : launch_mlp_fwd_t<T, 2, true, false>(m, s, nf, theta, af, acts, e_atom, nd))
                      : (wide ? launch_mlp_fwd_t<T, 2, false, true>(m, s, nf, theta, af, acts, e_atom, nd) : launch_mlp_fwd_t<T, 2, false, false>(m, s, nf, theta, af, acts, e_atom, nd));
    default: return wg ? (wide ? launch_mlp_fwd_t<T, 1, true, true>(m, s, nf, theta, af, acts, e_atom, nd) : launch_mlp_fwd_t<T, 1, true, false>(m, s, nf, theta, af, acts, e_atom, nd))
                       : (wide ? launch_mlp_fwd_t<T, 1, false, true>(m, s, nf, theta, af, acts, e_atom, nd) : launch_mlp_fwd_t<T, 1, false, false>(m, s, nf, theta, af, acts, e_atom, nd));
  }
}

template <class T>
static int launch_mlp_bwd(stafb_model* m, cudaStream_t s, int nf, const T* theta, const T* af, const T* acts,
                          const T* ebar, const T* u, T* gaf, T* grad) {
  if constexpr (std::is_same<T, float>::value) {
    if (m->mma) return launch_mlp_bwd_mma(m, s, nf, theta, af, acts, ebar, u, gaf, grad);
  }
  const bool wg = m->stage == 0, wide = m->md.maxw > 64;  // the dense products' form: see mlp.cuh
  switch (m->aw) {
    case 4: return wg ? (wide ? launch_mlp_bwd_t<T, 4, true, true>(m, s, nf, theta, af, acts, ebar, u, gaf, grad) : launch_mlp_bwd_t<T, 4, true, false>(m, s, nf, theta, af, acts, ebar, u, gaf, grad))
                      : (wide ? launch_mlp_bwd_t<T, 4, false, true>(m, s, nf, theta, af, acts, ebar, u, gaf, grad) : launch_mlp_bwd_t<T, 4, false, false>(m, s, nf, theta, af, acts, ebar, u, gaf, grad));
    case 2: return wg ? (wide ? launch_mlp_bwd_t<T, 2, true, true>(m, s, nf, theta, af, acts, ebar, u, gaf, grad) : launch_mlp_bwd_t<T, 2, true, false>(m, s, nf, theta, af, acts, ebar, u, gaf, grad))
                      : (wide ? launch_mlp_bwd_t<T, 2, false, true>(m, s, nf, theta, af, acts, ebar, u, gaf, grad) : launch_mlp_bwd_t<T, 2, false, false>(m, s, nf, theta, af, acts, ebar, u, gaf, grad));
    default: return wg ? (wide ? launch_mlp_bwd_t<T, 1, true, true>(m, s, nf, theta, af, acts, ebar, u, gaf, grad) : launch_mlp_bwd_t<T, 1, true, false>(m, s, nf, theta, af, acts, ebar, u, gaf, grad))
                       : (wide ? launch_mlp_bwd_t<T, 1, false, true>(m, s, nf, theta, af, acts, ebar, u, gaf, grad) : launch_mlp_bwd_t<T, 1, false, false>(m, s, nf, theta, af, acts, ebar, u, gaf, grad));
  }
}

// Domain mode of the fused path: one frame of nall atoms whose first N (the model's species-sorted
// atoms) are the centres; the rest are ghosts that only act as neighbours and receive forces.
struct DomainArgs {
  int nall;
  const int* tmap;     // device, [nall] species of every atom
  const int* howmany;  // device, [N] or null: caller-supplied neighbour list (no search, no minimum image)
  const int* with;     // device, [N, nr]
};

template <class T>
static int run_fused(stafb_ctx* c, stafb_model* m, cudaStream_t s, const T* pos, const T* box, int nf,
                     const T* theta, const T* emb, int per_atom, bool train, const T* e_label, const T* f_label,
                     double pe, double pf, double pb, double bound, int loss_kind, double* losses_out, T* grad,
                     T* energy_out, T* force_out, const DomainArgs* dom = nullptr, T* virial_out = nullptr,
                     const stafb_model::NlSet* pre = nullptr, const T* v_label = nullptr, double pv = 0.0) {
  if (!c || !m || (!pos && !pre) || !theta || !emb || nf <= 0) return STAFB_ERR_INVALID;
  if (!box && !pre && !(dom && dom->howmany)) return STAFB_ERR_INVALID;
  if (pre && (dom || pre->nf != nf)) return STAFB_ERR_INVALID;
  if (nf > c->max_batch) return STAFB_ERR_CAPACITY;
  if (train && (!e_label || !f_label || !grad || !losses_out)) return STAFB_ERR_INVALID;
  const ModelDev& d = m->md;
  const int N = d.N;
  if (dom && (nf != 1 || train || !dom->tmap || dom->nall < N || !force_out)) return STAFB_ERR_INVALID;
  const int nall = dom ? dom->nall : N;
  c->launches = 0;
  c->n_phase = 0;
  auto mark = [&]() {
    if (c->timing && c->n_phase < 16) cudaEventRecord(c->ev[c->n_phase++], s);
  };
  mark();
  void* rows = pre ? pre->rows : m->rows;
  const stafb_ctx* cg = pre ? pre->ctx : c;  // owner of the status word the neighbour kernels of this evaluation used
  int rc = STAFB_OK;
  if (pre) {
    c->launches = pre->ctx->launches;
  } else {
    const RowSink sk = row_sink(m, rows, dom ? dom->tmap : nullptr);
    if (dom && dom->howmany)
      rc = launch_rows_from_list<T>(c, s, pos, N, nall, dom->howmany, dom->with, &sk);
    else
      rc = launch_descriptors<T>(c, s, pos, box, nf, nall, (T*)nullptr, (T*)nullptr, (T*)nullptr, (int*)nullptr,
                                 (int*)nullptr, (T*)nullptr, (T*)nullptr, (T*)nullptr, (int*)nullptr, N, &sk);
  }
  if (rc != STAFB_OK) return rc;
  T* af = (T*)m->af; T* nd = (T*)m->nd; T* acts = (T*)m->acts; T* e_atom = (T*)m->e_atom;
  T* force = force_out ? force_out : (T*)m->force;
  T* energy = energy_out ? energy_out : (T*)m->energy;
  STAFB_CUDA_OK(launch_chained(
      k_prep<T>, 64, 256, 0, s, d, theta, emb, (T*)m->wpack, m->wstride, m->spar, m->sl.total, m->sl, (void*)force,
      sizeof(T) * (size_t)nf * 3 * nall,
      train ? (void*)grad : (void*)nullptr, train ? sizeof(T) * (size_t)m->n_params : (size_t)0, (void*)m->losses_d,
      sizeof(double) * ((virial_out || v_label) ? 8 + (1 + 9 * VIR_SLOTS) * (size_t)c->max_batch
                                                : 8 + (size_t)c->max_batch),
      train ? f_label : (const T*)nullptr, (T*)m->flab, train ? (size_t)nf * 3 * N : (size_t)0,
      m->mma ? (T*)m->wm : (T*)nullptr, m->wm_stride));
  c->launches++;
  mark();  // descriptors
  SweepCall<T> sc;
  memset(&sc, 0, sizeof(sc));
  sc.rows = rows; sc.nf = nf; sc.nall = nall; sc.status = cg->status_d;
  sc.out = af;
  sc.vout = train ? (T*)m->vrow : nullptr;
  rc = train ? launch_sweep<T, MODE_AFV>(m, s, sc) : launch_sweep<T, MODE_AF>(m, s, sc);
  if (rc != STAFB_OK) return rc;
  mark();  // af_fwd
  rc = launch_mlp_fwd<T>(m, s, nf, theta, af, acts, e_atom, nd);
  if (rc != STAFB_OK) return rc;
  mark();  // mlp_fwd
  if (v_label && !train) return STAFB_ERR_INVALID;
  double* vacc = (virial_out || v_label) ? m->losses_d + 8 + c->max_batch : nullptr;
  sc.chan_in = nd; sc.out = force; sc.vout = nullptr; sc.vir = vacc;
  rc = launch_sweep<T, MODE_FORCE>(m, s, sc);
  if (rc != STAFB_OK) return rc;
  mark();  // force
  if (train) {
    // the backward sweep of the forces forms dL/dF = pf/(3 nf N) * L'(F - F_label) per component itself, so the loss
    // kernel is off the path between the two sweeps and runs under this sweep's tail
    T* gradnet = (T*)m->gradnet;
    sc.chan_in = nd; sc.force = force; sc.flab = (const T*)m->flab; sc.loss_kind = loss_kind;
    sc.fscale = (T)pf / T((double)((size_t)nf * 3 * N));
    sc.out = gradnet; sc.grad = grad; sc.vir = nullptr;
    // with a virial loss its cotangent, pv/(9 nf) * L'(W - W_label), is formed on the fly as well
    sc.vacc = v_label ? vacc : nullptr; sc.vlab = v_label; sc.vscale = (T)(pv / (9.0 * nf));
    rc = launch_sweep<T, MODE_FGRAD>(m, s, sc);
    if (rc != STAFB_OK) return rc;
    mark();  // force_grad
  }
  {
    int fb = 0;
    if (train) {
      fb = (int)(((size_t)nf * 3 * N + 255) / 256);
      if (fb > 296) fb = 296;
    }
    // a large frame of an inference evaluation: its atomic energies summed by several blocks
    const int eb = train ? 1 : std::min(LOSS_EB_MAX, std::max(1, N / 1024));
    const int grid = nf * eb + fb + (train ? 1 : 0);
    STAFB_CUDA_OK(launch_chained(k_loss<T>, grid, 256, 0, s, d, nf, eb, fb, per_atom, train ? 1 : 0, e_atom, energy,
                                 e_label, force, (const T*)m->flab, theta, (T)pe, (T)pf, (T)pb, (T)bound, loss_kind,
                                 (T*)m->ebar, grad, m->losses_d, cg->status_d, c->status_d, vacc, virial_out,
                                 train ? m->mirror_next : (double*)nullptr, m->epart,
                                 reinterpret_cast<unsigned*>(m->epart + (size_t)c->max_batch * LOSS_EB_MAX), v_label,
                                 (T)pv));
    m->mirror_next = nullptr;
    c->launches++;
  }
  mark();  // loss
  if (train) {
    T* gaf = (T*)m->gaf;
    rc = launch_mlp_bwd<T>(m, s, nf, theta, af, acts, (const T*)m->ebar, (const T*)m->gradnet, gaf, grad);
    if (rc != STAFB_OK) return rc;
    mark();  // mlp_bwd
    if (losses_out != m->losses_d)
      STAFB_CUDA_OK(cudaMemcpyAsync(losses_out, m->losses_d, sizeof(double) * 4, cudaMemcpyDeviceToDevice, s));
    if (v_label && losses_out != m->losses_d)  // fifth loss of the energy + force + virial training
      STAFB_CUDA_OK(cudaMemcpyAsync(losses_out + 4, m->losses_d + 5, sizeof(double), cudaMemcpyDeviceToDevice, s));
  }
  STAFB_CUDA_OK(cudaGetLastError());
  return STAFB_OK;
}

// The MLP head alone on caller-supplied fingerprints: energy = 0.5 * sum of the atomic energies,
// dE_daf = d(sum of the atomic energies)/dAF - the convention of the reference's pluggable MLP
// (libstaf/include/staf_mlp.h:10-15).  af and dE_daf: [N][Fmax] rows in the model's atom order.
template <class T>
static int run_mlp_only(stafb_ctx* c, stafb_model* m, cudaStream_t s, const T* af, const T* theta, const T* emb,
                        T* energy, T* dE_daf) {
  const ModelDev& d = m->md;
  c->launches = 0;
  STAFB_CUDA_OK(launch_chained(k_prep<T>, 64, 256, 0, s, d, theta, emb, (T*)m->wpack, m->wstride, m->spar, m->sl.total,
                               m->sl, (void*)nullptr, (size_t)0, (void*)nullptr, (size_t)0, (void*)m->losses_d,
                               sizeof(double) * (8 + (size_t)c->max_batch), (const T*)nullptr, (T*)m->flab, (size_t)0,
                               m->mma ? (T*)m->wm : (T*)nullptr, m->wm_stride));
  c->launches++;
  int rc = launch_mlp_fwd<T>(m, s, 1, theta, af, (T*)m->acts, (T*)m->e_atom, dE_daf);
  if (rc != STAFB_OK) return rc;
  const int eb = std::min(LOSS_EB_MAX, std::max(1, d.N / 1024));
  // an ordinary launch: k_loss sums the atomic energies ahead of its chain wait, which is only right when the MLP
  // kernel is two kernels back (as in the fused sequences); here it is the direct predecessor
  k_loss<T><<<eb, 256, 0, s>>>(d, 1, eb, 0, 0, 0, (const T*)m->e_atom, energy, (const T*)nullptr, (const T*)nullptr,
                               (const T*)nullptr, theta, T(0), T(0), T(0), T(0), 0, (T*)m->ebar, (T*)nullptr,
                               m->losses_d, c->status_d, c->status_d, (const double*)nullptr, (T*)nullptr,
                               (double*)nullptr, m->epart,
                               reinterpret_cast<unsigned*>(m->epart + (size_t)c->max_batch * LOSS_EB_MAX),
                               (const T*)nullptr, T(0));
  c->launches++;
  STAFB_CUDA_OK(cudaGetLastError());
  return STAFB_OK;
}

extern "C" int stafb_mlp_eval(stafb_ctx* c, stafb_model* m, void* stream, const void* af_d, const void* theta,
                              const void* emb, void* energy_d, void* dE_daf_d) {
  if (!c || !m || !af_d || !theta || !emb || !energy_d || !dE_daf_d) return STAFB_ERR_INVALID;
  cudaStream_t s = (cudaStream_t)stream;
  if (c->dtype == STAFB_F32)
    return run_mlp_only<float>(c, m, s, (const float*)af_d, (const float*)theta, (const float*)emb, (float*)energy_d,
                               (float*)dE_daf_d);
  return run_mlp_only<double>(c, m, s, (const double*)af_d, (const double*)theta, (const double*)emb,
                              (double*)energy_d, (double*)dE_daf_d);
}

extern "C" int stafb_energy_force(stafb_ctx* c, stafb_model* m, void* stream, const void* pos, const void* box,
                                  int nf, const void* theta, const void* emb, int per_atom, void* energy,
                                  void* force) {
  if (!c || !m) return STAFB_ERR_INVALID;
  cudaStream_t s = (cudaStream_t)stream;
  if (c->dtype == STAFB_F32)
    return run_fused<float>(c, m, s, (const float*)pos, (const float*)box, nf, (const float*)theta,
                            (const float*)emb, per_atom, false, nullptr, nullptr, 0, 0, 0, 0, 0, nullptr, nullptr,
                            (float*)energy, (float*)force);
  return run_fused<double>(c, m, s, (const double*)pos, (const double*)box, nf, (const double*)theta,
                           (const double*)emb, per_atom, false, nullptr, nullptr, 0, 0, 0, 0, 0, nullptr, nullptr,
                           (double*)energy, (double*)force);
}

extern "C" int stafb_energy_force_domain(stafb_ctx* c, stafb_model* m, void* stream, const void* pos, const void* box,
                                         int nall, const int* type_map, const int* howmany, const int* with,
                                         const void* theta, const void* emb, void* energy, void* force,
                                         void* virial) {
  if (!c || !m || !type_map || (howmany && !with)) return STAFB_ERR_INVALID;
  if (nall > c->n_max) return STAFB_ERR_CAPACITY;
  cudaStream_t s = (cudaStream_t)stream;
  DomainArgs dom;
  dom.nall = nall; dom.tmap = type_map; dom.howmany = howmany; dom.with = with;
  if (c->dtype == STAFB_F32)
    return run_fused<float>(c, m, s, (const float*)pos, (const float*)box, 1, (const float*)theta, (const float*)emb,
                            0, false, nullptr, nullptr, 0, 0, 0, 0, 0, nullptr, nullptr, (float*)energy,
                            (float*)force, &dom, (float*)virial);
  return run_fused<double>(c, m, s, (const double*)pos, (const double*)box, 1, (const double*)theta,
                           (const double*)emb, 0, false, nullptr, nullptr, 0, 0, 0, 0, 0, nullptr, nullptr,
                           (double*)energy, (double*)force, &dom, (double*)virial);
}

extern "C" int stafb_energy_force_virial(stafb_ctx* c, stafb_model* m, void* stream, const void* pos, const void* box,
                                         int nf, const void* theta, const void* emb, int per_atom, void* energy,
                                         void* force, void* virial) {
  if (!c || !m) return STAFB_ERR_INVALID;
  cudaStream_t s = (cudaStream_t)stream;
  if (c->dtype == STAFB_F32)
    return run_fused<float>(c, m, s, (const float*)pos, (const float*)box, nf, (const float*)theta,
                            (const float*)emb, per_atom, false, nullptr, nullptr, 0, 0, 0, 0, 0, nullptr, nullptr,
                            (float*)energy, (float*)force, nullptr, (float*)virial);
  return run_fused<double>(c, m, s, (const double*)pos, (const double*)box, nf, (const double*)theta,
                           (const double*)emb, per_atom, false, nullptr, nullptr, 0, 0, 0, 0, 0, nullptr, nullptr,
                           (double*)energy, (double*)force, nullptr, (double*)virial);
}

extern "C" int stafb_train_step(stafb_ctx* c, stafb_model* m, void* stream, const void* pos, const void* box, int nf,
                                const void* theta, const void* emb, const void* el, const void* fl, double pe,
                                double pf, double pb, double bound, int loss_kind, double* losses_d, void* grad,
                                void* energy, void* force) {
  if (!c || !m) return STAFB_ERR_INVALID;
  cudaStream_t s = (cudaStream_t)stream;
  if (c->dtype == STAFB_F32)
    return run_fused<float>(c, m, s, (const float*)pos, (const float*)box, nf, (const float*)theta,
                            (const float*)emb, 1, true, (const float*)el, (const float*)fl, pe, pf, pb, bound,
                            loss_kind, losses_d, (float*)grad, (float*)energy, (float*)force);
  return run_fused<double>(c, m, s, (const double*)pos, (const double*)box, nf, (const double*)theta,
                           (const double*)emb, 1, true, (const double*)el, (const double*)fl, pe, pf, pb, bound,
                           loss_kind, losses_d, (double*)grad, (double*)energy, (double*)force);
}

// Energy + force + virial training evaluation (full_train_e_f_v, STAF/staf_models/staf_model.py:313-384): the
// loss gains pv * L(W - W_label), mean over [nf, 9], with W the virial of the ...Virial force operators.
// losses_d[5] = loss, loss_e, loss_bound, loss_f, loss_v.
extern "C" int stafb_train_step_virial(stafb_ctx* c, stafb_model* m, void* stream, const void* pos, const void* box,
                                       int nf, const void* theta, const void* emb, const void* el, const void* fl,
                                       const void* vl, double pe, double pf, double pv, double pb, double bound,
                                       int loss_kind, double* losses_d, void* grad, void* energy, void* force,
                                       void* virial) {
  if (!c || !m || !vl) return STAFB_ERR_INVALID;
  cudaStream_t s = (cudaStream_t)stream;
  if (c->dtype == STAFB_F32)
    return run_fused<float>(c, m, s, (const float*)pos, (const float*)box, nf, (const float*)theta,
                            (const float*)emb, 1, true, (const float*)el, (const float*)fl, pe, pf, pb, bound,
                            loss_kind, losses_d, (float*)grad, (float*)energy, (float*)force, nullptr, (float*)virial,
                            nullptr, (const float*)vl, pv);
  return run_fused<double>(c, m, s, (const double*)pos, (const double*)box, nf, (const double*)theta,
                           (const double*)emb, 1, true, (const double*)el, (const double*)fl, pe, pf, pb, bound,
                           loss_kind, losses_d, (double*)grad, (double*)energy, (double*)force, nullptr,
                           (double*)virial, nullptr, (const double*)vl, pv);
}

// Allocates neighbour-row set `slot` (0 or 1) of the model on first use.
static int ensure_nl(stafb_ctx* c, stafb_model* m, int slot) {
  stafb_model::NlSet& q = m->nl[slot];
  if (q.ctx) return STAFB_OK;
  int rc = stafb_create(&q.ctx, c->dtype, c->Rc, c->Rs, c->Ra, c->nr, c->na, c->n_max, c->max_batch);
  if (rc != STAFB_OK) { q.ctx = nullptr; return rc; }
  const size_t A = (size_t)c->max_batch * c->n_max;
  STAFB_CUDA_OK(cudaMalloc(&q.rows, A * (size_t)m->row_stride));
  STAFB_CUDA_OK(cudaMemset(q.rows, 0, A * (size_t)m->row_stride));
  STAFB_CUDA_OK(cudaEventCreateWithFlags(&q.ready, cudaEventDisableTiming));
  q.nf = 0;
  return STAFB_OK;
}

extern "C" int stafb_descriptors_prefetch(stafb_ctx* c, stafb_model* m, void* stream, const void* pos,
                                          const void* box, int nf, int slot) {
  if (!c || !m || !pos || !box || slot < 0 || slot > 1) return STAFB_ERR_INVALID;
  if (nf <= 0 || nf > c->max_batch) return STAFB_ERR_CAPACITY;
  int rc = ensure_nl(c, m, slot);
  if (rc != STAFB_OK) return rc;
  stafb_model::NlSet& q = m->nl[slot];
  cudaStream_t s = (cudaStream_t)stream;
  const int N = m->md.N;
  q.ctx->launches = 0;
  const RowSink sk = row_sink(m, q.rows, nullptr);
  if (c->dtype == STAFB_F32)
    rc = launch_descriptors<float>(q.ctx, s, (const float*)pos, (const float*)box, nf, N, (float*)nullptr,
                                   (float*)nullptr, (float*)nullptr, (int*)nullptr, (int*)nullptr, (float*)nullptr,
                                   (float*)nullptr, (float*)nullptr, (int*)nullptr, N, &sk);
  else
    rc = launch_descriptors<double>(q.ctx, s, (const double*)pos, (const double*)box, nf, N, (double*)nullptr,
                                    (double*)nullptr, (double*)nullptr, (int*)nullptr, (int*)nullptr,
                                    (double*)nullptr, (double*)nullptr, (double*)nullptr, (int*)nullptr, N, &sk);
  if (rc != STAFB_OK) return rc;
  q.nf = nf;
  STAFB_CUDA_OK(cudaGetLastError());
  return STAFB_OK;
}

// The step on the neighbour rows of `slot`; vl (device, [nf,9]) non-null adds the virial loss.
static int step_prefetched(stafb_ctx* c, stafb_model* m, void* stream, int slot, int nf, const void* theta,
                           const void* emb, const void* el, const void* fl, const void* vl, double pe, double pf,
                           double pv, double pb, double bound, int loss_kind, double* losses_d, void* grad,
                           void* energy, void* force) {
  if (!c || !m || slot < 0 || slot > 1 || !m->nl[slot].ctx) return STAFB_ERR_INVALID;
  cudaStream_t s = (cudaStream_t)stream;
  const stafb_model::NlSet* q = &m->nl[slot];
  if (c->dtype == STAFB_F32)
    return run_fused<float>(c, m, s, nullptr, nullptr, nf, (const float*)theta, (const float*)emb, 1, true,
                            (const float*)el, (const float*)fl, pe, pf, pb, bound, loss_kind, losses_d, (float*)grad,
                            (float*)energy, (float*)force, nullptr, nullptr, q, (const float*)vl, pv);
  return run_fused<double>(c, m, s, nullptr, nullptr, nf, (const double*)theta, (const double*)emb, 1, true,
                           (const double*)el, (const double*)fl, pe, pf, pb, bound, loss_kind, losses_d,
                           (double*)grad, (double*)energy, (double*)force, nullptr, nullptr, q, (const double*)vl,
                           pv);
}

extern "C" int stafb_train_step_prefetched(stafb_ctx* c, stafb_model* m, void* stream, int slot, int nf,
                                           const void* theta, const void* emb, const void* el, const void* fl,
                                           double pe, double pf, double pb, double bound, int loss_kind,
                                           double* losses_d, void* grad, void* energy, void* force) {
  return step_prefetched(c, m, stream, slot, nf, theta, emb, el, fl, nullptr, pe, pf, 0.0, pb, bound, loss_kind,
                         losses_d, grad, energy, force);
}

extern "C" int stafb_train_step_host(stafb_ctx* c, stafb_model* m, void* stream, const void* pos_h,
                                     const void* box_h, int nf, const void* theta, const void* emb,
                                     const void* el_h, const void* fl_h, double pe, double pf, double pb,
                                     double bound, int loss_kind, double* losses_h, void* grad);

// Pipelined form of stafb_train_step_host: _begin copies the host inputs into the slot's pinned block,
// enqueues ONE host->device copy, the step and the device->host copy of the losses and the status word, and
// returns without waiting; _end waits for that slot and hands the results over.  With two slots the host
// prepares step k+1 while the GPU runs step k.
static int host_step_begin(stafb_ctx* c, stafb_model* m, void* stream, const void* pos_h, const void* box_h, int nf,
                           const void* theta, const void* emb, const void* el_h, const void* fl_h, double pe,
                           double pf, double pb, double bound, int loss_kind, void* grad, int slot,
                           const void* vl_h = nullptr, double pv = 0.0) {
  if (!c || !m || !pos_h || !box_h || !el_h || !fl_h || slot < 0 || slot > 2) return STAFB_ERR_INVALID;
  if (nf <= 0 || nf > c->max_batch) return STAFB_ERR_CAPACITY;
  if (m->slot_busy[slot]) return STAFB_ERR_INVALID;  // the previous step of this slot has not been collected
  cudaStream_t s = (cudaStream_t)stream;
  const size_t es = m->es, A = (size_t)nf * m->md.N;
  const size_t o_fl = es * A * 3, o_box = o_fl + es * A * 3, o_el = o_box + es * (size_t)nf * 6;
  const size_t o_vl = o_el + es * (size_t)nf;
  char* ph = m->slot_in_h[slot];
  if (vl_h) memcpy(ph + o_vl, vl_h, es * (size_t)nf * 9);
  memcpy(ph, pos_h, es * A * 3);
  memcpy(ph + o_fl, fl_h, es * A * 3);
  memcpy(ph + o_box, box_h, es * (size_t)nf * 6);
  memcpy(ph + o_el, el_h, es * (size_t)nf);
  double* oh = m->slot_out_h[slot];
  // No copy-engine transfers on the stream: the kernels read the step's inputs directly from the slot's pinned
  // (device-mapped) block over PCIe - positions and box once in the cell-list kernel, the labels once in the
  // loss kernel - and the loss kernel writes the four losses and the status word straight into the slot's
  // pinned result block.  That takes one host->device and two device->host DMA latencies off every step.
  // Slots 0 and 1 build their neighbour rows on the model's side stream: the rows depend only on the positions,
  // so the GPU works on them while the main stream is still in the previous step (or in the caller's gradient
  // all-reduce and optimiser update); the rest of the step waits for them through an event.  Slot 2 (the
  // one-call form) runs everything on the caller's stream.
  const bool split = slot < 2;
  if (split) {
    if (!m->side) STAFB_CUDA_OK(cudaStreamCreateWithFlags(&m->side, cudaStreamNonBlocking));
    const int rc0 = ensure_nl(c, m, slot);
    if (rc0 != STAFB_OK) return rc0;
  }
  auto enqueue_rows = [&]() -> int {
    return stafb_descriptors_prefetch(c, m, m->side, ph, ph + o_box, nf, slot);
  };
  auto enqueue = [&]() -> int {
    // the virial labels are read by every block of the force-backward sweep: one small copy to the device
    // instead of reads over PCIe (the other labels are read once, by the loss kernel and the preparation kernel)
    if (vl_h &&
        cudaMemcpyAsync(m->vlab_d, ph + o_vl, es * (size_t)nf * 9, cudaMemcpyHostToDevice, s) != cudaSuccess)
      return STAFB_ERR_CUDA;
    m->mirror_next = oh;
    if (split)
      return step_prefetched(c, m, stream, slot, nf, theta, emb, ph + o_el, ph + o_fl, vl_h ? m->vlab_d : nullptr, pe,
                             pf, pv, pb, bound, loss_kind, m->losses_d, grad, nullptr, nullptr);
    if (vl_h)
      return stafb_train_step_virial(c, m, stream, ph, ph + o_box, nf, theta, emb, ph + o_el, ph + o_fl, m->vlab_d, pe,
                                     pf, pv, pb, bound, loss_kind, m->losses_d, grad, nullptr, nullptr, nullptr);
    return stafb_train_step(c, m, stream, ph, ph + o_box, nf, theta, emb, ph + o_el, ph + o_fl, pe, pf, pb, bound,
                            loss_kind, m->losses_d, grad, nullptr, nullptr);
  };
  // The same call signature on the same slot is first run as plain launches (which also performs the one-time
  // kernel attribute set-up), then captured into CUDA graphs (one for the rows, one for the rest), then replayed:
  // two launches per step instead of fourteen.  All addresses inside the graphs are the slot's own buffers and
  // the caller's theta/emb/grad.
  stafb_model::SlotKey key;
  memset(&key, 0, sizeof(key));
  key.nf = nf; key.loss_kind = loss_kind; key.theta = theta; key.emb = emb; key.grad = grad; key.stream = stream;
  key.pe = pe; key.pf = pf; key.pb = pb; key.bound = bound; key.pv = pv; key.with_v = vl_h != nullptr;
  const bool same = m->slot_state[slot] != 0 && memcmp(&key, &m->slot_key[slot], sizeof(key)) == 0;
  if (!same) {
    if (m->slot_exec[slot]) { cudaGraphExecDestroy(m->slot_exec[slot]); m->slot_exec[slot] = nullptr; }
    if (split && m->nl_exec[slot]) { cudaGraphExecDestroy(m->nl_exec[slot]); m->nl_exec[slot] = nullptr; }
    m->slot_key[slot] = key;
    m->slot_state[slot] = 0;
  }
  static const bool no_graph = getenv("STAFB_NO_STEP_GRAPH") != nullptr;
  // captures what `fn` enqueues on `cs` into an executable graph; false (and a cleared error) if that fails
  auto capture = [&](cudaStream_t cs, cudaGraphExec_t* exec, auto&& fn) -> bool {
    cudaGraph_t g = nullptr;
    bool ok = cudaStreamBeginCapture(cs, cudaStreamCaptureModeThreadLocal) == cudaSuccess;
    if (ok) {
      const int rcc = fn();
      ok = cudaStreamEndCapture(cs, &g) == cudaSuccess && rcc == STAFB_OK && g != nullptr;
    }
    if (ok) ok = cudaGraphInstantiate(exec, g, 0) == cudaSuccess;
    if (g) cudaGraphDestroy(g);
    if (!ok) { cudaGetLastError(); *exec = nullptr; }
    return ok;
  };
  if (m->slot_state[slot] == 1 && !c->timing && !no_graph) {
    bool ok = capture(s, &m->slot_exec[slot], enqueue);
    if (ok && split) ok = capture(m->side, &m->nl_exec[slot], enqueue_rows);
    if (!ok) {
      if (m->slot_exec[slot]) { cudaGraphExecDestroy(m->slot_exec[slot]); m->slot_exec[slot] = nullptr; }
      m->mirror_next = nullptr;
    }
    m->slot_state[slot] = ok ? 2 : -1;  // -1: plain launches for this signature from now on
  } else if (m->slot_state[slot] == 0) {
    m->slot_state[slot] = 1;
  }
  const bool replay = m->slot_state[slot] == 2;
  int rc = STAFB_OK;
  if (split) {
    if (replay) STAFB_CUDA_OK(cudaGraphLaunch(m->nl_exec[slot], m->side));
    else if ((rc = enqueue_rows()) != STAFB_OK) return rc;
    STAFB_CUDA_OK(cudaEventRecord(m->nl[slot].ready, m->side));
    STAFB_CUDA_OK(cudaStreamWaitEvent(s, m->nl[slot].ready, 0));
  }
  if (replay) STAFB_CUDA_OK(cudaGraphLaunch(m->slot_exec[slot], s));
  else if ((rc = enqueue()) != STAFB_OK) return rc;
  STAFB_CUDA_OK(cudaEventRecord(m->slot_done[slot], s));
  m->slot_busy[slot] = 1;
  return STAFB_OK;
}

extern "C" int stafb_train_step_host_begin(stafb_ctx* c, stafb_model* m, void* stream, const void* pos_h,
                                           const void* box_h, int nf, const void* theta, const void* emb,
                                           const void* el_h, const void* fl_h, double pe, double pf, double pb,
                                           double bound, int loss_kind, void* grad, int slot) {
  if (slot < 0 || slot > 1) return STAFB_ERR_INVALID;
  return host_step_begin(c, m, stream, pos_h, box_h, nf, theta, emb, el_h, fl_h, pe, pf, pb, bound, loss_kind, grad,
                         slot);
}

static int host_step_end(stafb_ctx* c, stafb_model* m, int slot, double* losses_h, bool with_v = false) {
  if (!c || !m || !losses_h || slot < 0 || slot > 2 || !m->slot_busy[slot]) return STAFB_ERR_INVALID;
  STAFB_CUDA_OK(cudaEventSynchronize(m->slot_done[slot]));
  m->slot_busy[slot] = 0;
  const double* oh = m->slot_out_h[slot];
  for (int q = 0; q < 4; q++) losses_h[q] = oh[q];
  if (with_v) losses_h[4] = oh[5];
  return *reinterpret_cast<const int*>(oh + 4);
}

extern "C" int stafb_train_step_host_end(stafb_ctx* c, stafb_model* m, int slot, double* losses_h) {
  if (slot < 0 || slot > 1) return STAFB_ERR_INVALID;
  return host_step_end(c, m, slot, losses_h);
}

// The same pair for the energy + force + virial step: vl_h [nf,9] host virial labels; losses_h[5] = loss, loss_e,
// loss_bound, loss_f, loss_v.
extern "C" int stafb_train_step_virial_host_begin(stafb_ctx* c, stafb_model* m, void* stream, const void* pos_h,
                                                  const void* box_h, int nf, const void* theta, const void* emb,
                                                  const void* el_h, const void* fl_h, const void* vl_h, double pe,
                                                  double pf, double pv, double pb, double bound, int loss_kind,
                                                  void* grad, int slot) {
  if (slot < 0 || slot > 1 || !vl_h) return STAFB_ERR_INVALID;
  return host_step_begin(c, m, stream, pos_h, box_h, nf, theta, emb, el_h, fl_h, pe, pf, pb, bound, loss_kind, grad,
                         slot, vl_h, pv);
}

extern "C" int stafb_train_step_virial_host_end(stafb_ctx* c, stafb_model* m, int slot, double* losses_h) {
  if (slot < 0 || slot > 1) return STAFB_ERR_INVALID;
  return host_step_end(c, m, slot, losses_h, true);
}


// The one-call form: the same staging and result path on a slot of its own, then wait.
extern "C" int stafb_train_step_host(stafb_ctx* c, stafb_model* m, void* stream, const void* pos_h,
                                     const void* box_h, int nf, const void* theta, const void* emb,
                                     const void* el_h, const void* fl_h, double pe, double pf, double pb,
                                     double bound, int loss_kind, double* losses_h, void* grad) {
  if (!losses_h) return STAFB_ERR_INVALID;
  const int rc = host_step_begin(c, m, stream, pos_h, box_h, nf, theta, emb, el_h, fl_h, pe, pf, pb, bound, loss_kind,
                                 grad, 2);
  if (rc != STAFB_OK) return rc;
  return host_step_end(c, m, 2, losses_h);
}

extern "C" int stafb_adam_step(stafb_ctx* c, void* stream, void* theta, const void* grad, void* mm, void* vv, int n,
                               double lr, double b1, double b2, double eps, int step, double gscale) {
  if (!c || !theta || !grad || !mm || !vv || n <= 0 || step < 1) return STAFB_ERR_INVALID;
  cudaStream_t s = (cudaStream_t)stream;
  // Keras Adam: lr_t = lr * sqrt(1-b2^t)/(1-b1^t); theta -= lr_t * m/(sqrt(v)+eps)
  const double lr_t = lr * sqrt(1.0 - pow(b2, (double)step)) / (1.0 - pow(b1, (double)step));
  if (c->dtype == STAFB_F32)
    k_adam<float><<<(n + 255) / 256, 256, 0, s>>>(n, (float*)theta, (const float*)grad, (float*)mm, (float*)vv,
                                                  (float)lr_t, (float)b1, (float)b2, (float)eps, (float)gscale);
  else
    k_adam<double><<<(n + 255) / 256, 256, 0, s>>>(n, (double*)theta, (const double*)grad, (double*)mm, (double*)vv,
                                                   lr_t, b1, b2, eps, gscale);
  STAFB_CUDA_OK(cudaGetLastError());
  return STAFB_OK;
}

extern "C" int stafb_adam_step_dev(stafb_ctx* c, void* stream, void* theta, const void* grad, void* mm, void* vv,
                                   int n, double lr, double b1, double b2, double eps, int* step_d, double gscale) {
  if (!c || !theta || !grad || !mm || !vv || n <= 0 || !step_d) return STAFB_ERR_INVALID;
  cudaStream_t s = (cudaStream_t)stream;
  if (c->dtype == STAFB_F32)
    STAFB_CUDA_OK(launch_chained(k_adam_dev<float>, (n + 255) / 256, 256, 0, s, n, (float*)theta, (const float*)grad,
                                 (float*)mm, (float*)vv, lr, b1, b2, (float)eps, (float)gscale, step_d));
  else
    STAFB_CUDA_OK(launch_chained(k_adam_dev<double>, (n + 255) / 256, 256, 0, s, n, (double*)theta,
                                 (const double*)grad, (double*)mm, (double*)vv, lr, b1, b2, eps, gscale, step_d));
  STAFB_CUDA_OK(cudaGetLastError());
  return STAFB_OK;
}
