// Per-species MLP energy head of the fused path (included by fused.cu inside namespace stafb).
//
// x = log(AF+1e-3) - mu ; Dense(tanh)... Dense(1)  (staf_models/staf_model.py:188-191,
// libstaf/src/mlp/staf_mlp_ort.cc:196-242 of the reference).  A block of 256 threads owns TA = 8*APT
// atoms of one species.  Every per-atom vector lives in shared memory feature-major ([feature][atom],
// row stride TA+4 words) and every Dense layer is staged in shared memory once per block; the
// matrix products are register-tiled so that one shared-memory load feeds several FMAs:
//   forward   thread = 4 outputs x 2 atoms : one 16-byte weight load + one atom-pair load -> 8 FMA
//   backward  thread = 1 input x 4 atoms   : one 16-byte weight load + four atom-quad loads -> 16 FMA
//   dL/dW     thread = 2 inputs x 2 outputs, atoms four at a time
// The weight row stride is chosen = 4 (mod 32) words, which makes both the forward pattern (lanes on
// consecutive output groups) and the backward pattern (lanes on consecutive inputs) conflict-free.
#pragma once
#include <cuda_pipeline.h>

constexpr int ML_PAD = 4;  // padding of the [feature][atom] rows, in words

// Optional phase clocks (build with -DSTAFB_SWEEP_CLOCKS): thread 0 of every block adds the clock64() ticks
// between consecutive ML_TICK marks to g_mlp_clk[kernel][phase]; read with stafb_mlp_clocks().
#ifdef STAFB_SWEEP_CLOCKS
__device__ unsigned long long g_mlp_clk[2][16];
#define ML_CLK_INIT long long mclk__ = clock64();
#define ML_TICK(k, p)                                                                              \
  {                                                                                                \
    const long long now__ = clock64();                                                             \
    if (threadIdx.x == 0) atomicAdd(&g_mlp_clk[k][p], (unsigned long long)(now__ - mclk__));       \
    mclk__ = now__;                                                                                \
  }
#else
#define ML_CLK_INIT
#define ML_TICK(k, p)
#endif

// row stride of a staged layer with `out` columns: smallest value >= out that is 4 mod 32
__host__ __device__ inline int ml_ld(int out) { return ((out + 27) / 32) * 32 + 4; }

template <class T>
struct LayerView {
  const T* W;  // element (i,j) at W[i*ld + j]
  const T* B;  // bias
  int ld;
  bool vec;    // rows are 16-byte aligned and padded with zeros up to a multiple of four columns
};

// The Dense layers reach the MLP kernels through a packed copy of the weights (k_prep writes it at the start
// of every evaluation, theta changes with every optimizer step): per species, the layers back to back, each
// as (in + 1) rows of ml_ld(out) words - weights [in][out] zero-padded to the row stride, then the bias row.
// That layout is exactly what the kernels want in shared memory, 16-byte aligned, so staging is a plain run
// of 16-byte asynchronous global->shared copies (all in flight together, no per-element address arithmetic).
__host__ __device__ inline int ml_layer_words(int in, int out) { return (in + 1) * ml_ld(out); }

template <class T>
__device__ __forceinline__ void stage_words(const T* __restrict__ src, T* wsm, int words) {
  constexpr int PER = 16 / (int)sizeof(T);  // elements per 16-byte copy; words is a multiple of 4
  for (int idx = threadIdx.x * PER; idx < words; idx += ML_THREADS * PER)
    __pipeline_memcpy_async(wsm + idx, src + idx, 16);
  __pipeline_commit();
}

__device__ __forceinline__ void ml_stage_wait() {
  __pipeline_wait_prior(0);
  __syncthreads();
}

template <class T>
__device__ __forceinline__ LayerView<T> layer_view(int in, int out, const T* base) {
  LayerView<T> v;
  v.ld = ml_ld(out);
  v.W = base; v.B = base + in * v.ld; v.vec = true;
  return v;
}

// Dense layer l of species t for the products below; wp = the species' packed weights in global memory.
// mode 2: every layer was staged when the kernel started (wsm holds them back to back); mode 1: stage this
// layer now; mode 0: read the packed copy in global memory (the layer does not fit next to the activations).
template <class T>
__device__ __forceinline__ LayerView<T> get_layer(const ModelDev& md, int t, int l, const T* __restrict__ wp, T* wsm,
                                                 int mode) {
  const int in = md.in_of(t, l), out = md.width[l];
  int off = 0;
  for (int k = 0; k < l; k++) off += ml_layer_words(md.in_of(t, k), md.width[k]);
  if (mode == 2) return layer_view<T>(in, out, wsm + off);
  __syncthreads();  // previous users of wsm are done, inputs of the layer are complete
  if (mode == 0) return layer_view<T>(in, out, wp + off);
  stage_words<T>(wp + off, wsm, ml_layer_words(in, out));
  ml_stage_wait();
  return layer_view<T>(in, out, wsm);
}

// mode 2: issue the copies of every layer (the caller overlaps them with its own global loads, then waits)
template <class T>
__device__ __forceinline__ void stage_all_layers(const ModelDev& md, int t, const T* __restrict__ wp, T* wsm) {
  int words = 0;
  for (int l = 0; l < md.n_dense; l++) words += ml_layer_words(md.in_of(t, l), md.width[l]);
  stage_words<T>(wp, wsm, words);
}

// Y[j][a] = act( b[j] + sum_i X[i][a] W[i,j] ).  A thread owns one output j for a group of eight atoms and
// one slice of the input range: the sum over i is split KS ways across adjacent lanes (so that all 256
// threads work even when the layer is narrow and the dependent FMA chains stay short) and the slices are
// combined with shuffles.
template <class T, int TA, bool TANH, bool BIAS>
__device__ __forceinline__ void dense_fwd(int in, int out, const LayerView<T> lv, const T* X, T* Y) {
  typedef typename Vec4<T>::type T4;
  constexpr int TAP = TA + ML_PAD, NO = TA / 8;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, ld = lv.ld;
  int KS = 1;
  while (KS < 32 && out * NO * KS < ML_THREADS && KS * 2 <= in) KS <<= 1;
  const int JL = 32 / KS, njg = (out + JL - 1) / JL;
  const int ks = lane & (KS - 1), jl = lane / KS;
  for (int item = warp; item < njg * NO; item += ML_THREADS / 32) {
    const int jg = item % njg, a0 = (item / njg) * 8;
    const int j = jg * JL + jl;
    T acc[8];
#pragma unroll
    for (int q = 0; q < 8; q++) acc[q] = T(0);
    if (j < out) {
#pragma unroll 4
      for (int i = ks; i < in; i += KS) {
        const T w = lv.W[i * ld + j];
        const T4 x0 = *reinterpret_cast<const T4*>(X + i * TAP + a0);
        const T4 x1 = *reinterpret_cast<const T4*>(X + i * TAP + a0 + 4);
        acc[0] += x0.x * w; acc[1] += x0.y * w; acc[2] += x0.z * w; acc[3] += x0.w * w;
        acc[4] += x1.x * w; acc[5] += x1.y * w; acc[6] += x1.z * w; acc[7] += x1.w * w;
      }
    }
    for (int off = 1; off < KS; off <<= 1) {
#pragma unroll
      for (int q = 0; q < 8; q++) acc[q] += __shfl_xor_sync(0xffffffffu, acc[q], off);
    }
    if (j < out && ks == 0) {
      const T bj = BIAS ? lv.B[j] : T(0);
      T4 y0, y1;
      y0.x = acc[0] + bj; y0.y = acc[1] + bj; y0.z = acc[2] + bj; y0.w = acc[3] + bj;
      y1.x = acc[4] + bj; y1.y = acc[5] + bj; y1.z = acc[6] + bj; y1.w = acc[7] + bj;
      if (TANH) {
        y0.x = r_tanh(y0.x); y0.y = r_tanh(y0.y); y0.z = r_tanh(y0.z); y0.w = r_tanh(y0.w);
        y1.x = r_tanh(y1.x); y1.y = r_tanh(y1.y); y1.z = r_tanh(y1.z); y1.w = r_tanh(y1.w);
      }
      *reinterpret_cast<T4*>(Y + j * TAP + a0) = y0;
      *reinterpret_cast<T4*>(Y + j * TAP + a0 + 4) = y1;
    }
  }
}

// Xo[i][a] = sum_j D[j][a] W[i,j]  (and the same for a second cotangent D2 -> Xo2 when given).  A thread
// owns one input i for a group of eight atoms and one slice of the output range (quads of outputs dealt
// KS <= 4 ways); lanes of a quarter-warp sit on consecutive inputs, which makes the 16-byte weight loads
// conflict-free with the row stride of ml_ld().
template <class T, int TA>
__device__ __forceinline__ void dense_bwd(int in, int out, const LayerView<T> lv, const T* D, T* Xo, const T* D2,
                                          T* Xo2) {
  typedef typename Vec4<T>::type T4;
  constexpr int TAP = TA + ML_PAD, NO = TA / 8;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, ld = lv.ld;
  const int nq = (out + 3) >> 2;
  int KS = 1;
  while (KS < 4 && in * NO * KS < ML_THREADS && KS * 2 <= nq) KS <<= 1;
  const int IL = 32 / KS, nig = (in + IL - 1) / IL;
  const int il = lane & (IL - 1), ks = lane / IL;
  __syncthreads();
  for (int item = warp; item < nig * NO; item += ML_THREADS / 32) {
    const int ig = item % nig, a0 = (item / nig) * 8;
    const int i = ig * IL + il;
    T a[8], b[8];
#pragma unroll
    for (int q = 0; q < 8; q++) a[q] = b[q] = T(0);
    auto fma8 = [&](T* s, const T w, const T* src) {
      const T4 d0 = *reinterpret_cast<const T4*>(src), d1 = *reinterpret_cast<const T4*>(src + 4);
      s[0] += w * d0.x; s[1] += w * d0.y; s[2] += w * d0.z; s[3] += w * d0.w;
      s[4] += w * d1.x; s[5] += w * d1.y; s[6] += w * d1.z; s[7] += w * d1.w;
    };
    if (i < in) {
      for (int q4 = ks; q4 < nq; q4 += KS) {
        const int j = q4 * 4;
        T wv[4];
        if (lv.vec) {
          const T4 w = *reinterpret_cast<const T4*>(lv.W + i * ld + j);  // padding columns are zero
          wv[0] = w.x; wv[1] = w.y; wv[2] = w.z; wv[3] = w.w;
        } else {
#pragma unroll
          for (int r = 0; r < 4; r++) wv[r] = (j + r < out) ? lv.W[i * ld + j + r] : T(0);
        }
#pragma unroll
        for (int r = 0; r < 4; r++) {
          if (j + r < out) {
            fma8(a, wv[r], D + (j + r) * TAP + a0);
            if (D2) fma8(b, wv[r], D2 + (j + r) * TAP + a0);
          }
        }
      }
    }
    for (int off = IL; off < 32; off <<= 1) {
#pragma unroll
      for (int q = 0; q < 8; q++) {
        a[q] += __shfl_xor_sync(0xffffffffu, a[q], off);
        if (D2) b[q] += __shfl_xor_sync(0xffffffffu, b[q], off);
      }
    }
    if (i < in && ks == 0) {
      T4 o;
      o.x = a[0]; o.y = a[1]; o.z = a[2]; o.w = a[3];
      *reinterpret_cast<T4*>(Xo + i * TAP + a0) = o;
      o.x = a[4]; o.y = a[5]; o.z = a[6]; o.w = a[7];
      *reinterpret_cast<T4*>(Xo + i * TAP + a0 + 4) = o;
      if (D2) {
        o.x = b[0]; o.y = b[1]; o.z = b[2]; o.w = b[3];
        *reinterpret_cast<T4*>(Xo2 + i * TAP + a0) = o;
        o.x = b[4]; o.y = b[5]; o.z = b[6]; o.w = b[7];
        *reinterpret_cast<T4*>(Xo2 + i * TAP + a0 + 4) = o;
      }
    }
  }
  __syncthreads();
}

// global row of atom slot a of this block (species t, first species-local index q0), or -1 past the end
__device__ __forceinline__ long long ml_atom_row(const ModelDev& md, int t, int q0, int nat, int a) {
  const int q = q0 + a;
  if (q >= nat) return -1;
  const int b = q / md.tipos[t];
  return (long long)b * md.N + md.shift[t] + (q - b * md.tipos[t]);
}

template <class T, int APT>
__global__ void __launch_bounds__(ML_THREADS)
    k_mlp_fwd(ModelDev md, int nf, const T* __restrict__ theta, const T* __restrict__ wpack, int wstride,
              const T* __restrict__ af, T* __restrict__ acts, T* __restrict__ e_atom, T* __restrict__ netderiv,
              double* __restrict__ e_sum /*[nf] accumulated*/, int stage) {
  constexpr int TA = 8 * APT, TAP = TA + ML_PAD;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __shared__ long long rows[TA];
  int t, q0;
  locate_block(md, nf, TA, t, q0);
  const int nat = nf * md.tipos[t];
  const int F = md.Fr[t] + md.Fa[t], Lq = md.n_dense, Fm = md.Fmax, Hs = md.Hsum, mw = md.maxw;
  T* X = reinterpret_cast<T*>(smem_raw);  // [Fm][TAP]
  T* H = X + Fm * TAP;                    // [Hs][TAP]
  T* C0 = H + Hs * TAP;                   // [mw][TAP]
  T* C1 = C0 + mw * TAP;                  // [mw][TAP]
  T* wsm = C1 + mw * TAP;                 // one staged layer
  const T* mu = theta + md.off_mu[t];
  const T* w = wpack + (size_t)t * wstride;  // this species' packed layers
  ML_CLK_INIT
  if (threadIdx.x < TA) rows[threadIdx.x] = ml_atom_row(md, t, q0, nat, threadIdx.x);
  if (stage == 2) stage_all_layers<T>(md, t, w, wsm);
  chain_wait();  // the packed weights are older than the preceding kernel; everything read below is its output
  __syncthreads();
  ML_TICK(0, 0)
  for (int idx = threadIdx.x; idx < F * TA; idx += ML_THREADS) {
    const int i = idx % F, a = idx / F;  // consecutive threads read consecutive fingerprints of one atom
    const long long gi = rows[a];
    X[i * TAP + a] = gi >= 0 ? r_log(af[gi * Fm + i] + T(1e-3)) - mu[i] : T(0);
  }
  ML_TICK(0, 1)
  if (stage == 2) ml_stage_wait();
  ML_TICK(0, 2)
  const T* hin = X;
  LayerView<T> lv;
  for (int l = 0; l < Lq; l++) {
    const int in = md.in_of(t, l), out = md.width[l];
    lv = get_layer<T>(md, t, l, w, wsm, stage);
    if (stage == 2) __syncthreads();  // the layer's input is complete
    T* hout = H + md.h_off(l) * TAP;
    if (l < Lq - 1) dense_fwd<T, TA, true, true>(in, out, lv, hin, hout);
    else dense_fwd<T, TA, false, true>(in, out, lv, hin, hout);
    hin = hout;
    ML_TICK(0, 3 + (l < 3 ? l : 3))
  }
  __syncthreads();
  // activations, block-local feature-major copy for the backward kernel
  T* ab = acts + (size_t)blockIdx.x * Hs * TA;
  for (int idx = threadIdx.x; idx < Hs * TA; idx += ML_THREADS) ab[idx] = H[(idx / TA) * TAP + (idx % TA)];
  if (threadIdx.x < TA) {
    const long long gi = rows[threadIdx.x];
    if (gi >= 0) e_atom[gi] = H[md.h_off(Lq - 1) * TAP + threadIdx.x];
  }
  if (threadIdx.x == 0) {
    // per-frame sums of the block's atomic energies (a block's atoms are consecutive: one or two frames)
    const T* eo = H + md.h_off(Lq - 1) * TAP;
    double acc = 0.0;
    long long bcur = -1;
    for (int a = 0; a < TA; a++) {
      const long long gi = rows[a];
      if (gi < 0) break;
      const long long b = gi / md.N;
      if (b != bcur) {
        if (bcur >= 0) atomicAdd(e_sum + bcur, acc);
        acc = 0.0;
        bcur = b;
      }
      acc += (double)eo[a];
    }
    if (bcur >= 0) atomicAdd(e_sum + bcur, acc);
  }
  ML_TICK(0, 7)
  // de/dx by the reverse sweep: cn = cotangent on the output of layer l
  T* cn = C0;
  T* cp = C1;
  if (threadIdx.x < TA) cn[threadIdx.x] = T(1);
  for (int l = Lq - 1; l >= 0; l--) {
    const int in = md.in_of(t, l), out = md.width[l];
    if (l < Lq - 1 || stage == 2) lv = get_layer<T>(md, t, l, w, wsm, stage);  // else: the last layer is still staged
    __syncthreads();
    if (l < Lq - 1) {
      const T* hl = H + md.h_off(l) * TAP;
      for (int idx = threadIdx.x; idx < out * TA; idx += ML_THREADS) {
        const int o = (idx / TA) * TAP + (idx % TA);
        cn[o] *= (T(1) - hl[o] * hl[o]);
      }
    }
    dense_bwd<T, TA>(in, out, lv, cn, cp, nullptr, nullptr);
    T* tmp = cn; cn = cp; cp = tmp;
    ML_TICK(0, 8 + (l < 3 ? l : 3))
  }
  for (int idx = threadIdx.x; idx < Fm * TA; idx += ML_THREADS) {
    const int i = idx % Fm, a = idx / Fm;
    const long long gi = rows[a];
    if (gi >= 0) netderiv[gi * Fm + i] = (i < F) ? cn[i * TAP + a] / (af[gi * Fm + i] + T(1e-3)) : T(0);
  }
  ML_TICK(0, 12)
}

// Backward of  S = sum_a ebar[a]*e[a] + sum_{a,c} u[a,c]*netderiv[a,c]  with respect to the
// weights, mu and AF: the first term is plain back-propagation, the second is the derivative
// of a directional derivative (tangent v = u/(AF+eps) pushed forward, then reversed) - what
// TensorFlow's autodiff does through grad_ene for the force loss (staf_model.py:191,225-228).
// The kernel also contracts dL/dAF with the per-atom d(AF)/d(alpha) rows left by the AF sweep
// (vrow), which yields the fingerprint part of dL/dalpha without another sweep over the triplets.
template <class T, int APT>
__global__ void __launch_bounds__(ML_THREADS)
    k_mlp_bwd(ModelDev md, int nf, const T* __restrict__ theta, const T* __restrict__ wpack, int wstride,
              const T* __restrict__ af, const T* __restrict__ acts, const T* __restrict__ ebar /*[nf]*/, const T* __restrict__ u /*[nf,N,Fmax]*/,
              const T* __restrict__ vrow /*[nf,N,nv] or null*/, int nv, T* __restrict__ gaf, T* __restrict__ grad,
              int stage) {
  typedef typename Vec4<T>::type T4;
  constexpr int TA = 8 * APT, TAP = TA + ML_PAD;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __shared__ long long rows[TA];
  int t, q0;
  locate_block(md, nf, TA, t, q0);
  const int nat = nf * md.tipos[t];
  const int F = md.Fr[t] + md.Fa[t], Lq = md.n_dense, Fm = md.Fmax, Hs = md.Hsum, mw = md.maxw;
  T* X = reinterpret_cast<T*>(smem_raw);  // [Fm][TAP] x
  T* V = X + Fm * TAP;                    // [Fm][TAP] tangent on x
  T* H = V + Fm * TAP;                    // [Hs][TAP] activations
  T* HD = H + Hs * TAP;                   // tangents of the activations
  T* AD = HD + Hs * TAP;                  // tangents of the pre-activations
  T* DQ = AD + Hs * TAP;                  // cotangent on the pre-activation (first-order channel)
  T* DP = DQ + Hs * TAP;                  // cotangent on the pre-activation tangent
  T* CQ = DP + Hs * TAP;                  // [mw][TAP]
  T* CP = CQ + mw * TAP;                  // [mw][TAP]
  T* wsm = CP + mw * TAP;                 // one staged layer
  const T* mu = theta + md.off_mu[t];
  const T* w = wpack + (size_t)t * wstride;  // this species' packed layers
  ML_CLK_INIT
  if (threadIdx.x < TA) rows[threadIdx.x] = ml_atom_row(md, t, q0, nat, threadIdx.x);
  if (stage == 2) stage_all_layers<T>(md, t, w, wsm);
  chain_wait();  // the packed weights are older than the preceding kernel; everything read below is its output
  __syncthreads();
  for (int idx = threadIdx.x; idx < F * TA; idx += ML_THREADS) {
    const int i = idx % F, a = idx / F;
    const long long gi = rows[a];
    T xv = T(0), vv = T(0);
    if (gi >= 0) {
      const T den = af[gi * Fm + i] + T(1e-3);
      xv = r_log(den) - mu[i];
      vv = u[gi * Fm + i] / den;
    }
    X[i * TAP + a] = xv;
    V[i * TAP + a] = vv;
  }
  const T* ab = acts + (size_t)blockIdx.x * Hs * TA;
  for (int idx = threadIdx.x; idx < Hs * TA; idx += ML_THREADS) {
    const int a = idx % TA;
    H[(idx / TA) * TAP + a] = (q0 + a < nat) ? ab[idx] : T(0);
  }
  if (stage == 2) ml_stage_wait();
  ML_TICK(1, 0)
  // forward tangent: AD = HDin W ; HD = AD * act'
  const T* hdin = V;
  LayerView<T> lv;
  for (int l = 0; l < Lq; l++) {
    const int in = md.in_of(t, l), out = md.width[l];
    lv = get_layer<T>(md, t, l, w, wsm, stage);
    if (stage == 2) __syncthreads();  // the layer's input is complete
    T* ado = AD + md.h_off(l) * TAP;
    T* hdo = HD + md.h_off(l) * TAP;
    dense_fwd<T, TA, false, false>(in, out, lv, hdin, ado);
    __syncthreads();
    const T* ho = H + md.h_off(l) * TAP;
    for (int idx = threadIdx.x; idx < out * TA; idx += ML_THREADS) {
      const int o = (idx / TA) * TAP + (idx % TA);
      hdo[o] = (l < Lq - 1) ? ado[o] * (T(1) - ho[o] * ho[o]) : ado[o];
    }
    hdin = hdo;
  }
  __syncthreads();
  ML_TICK(1, 1)
  // reverse over (h, hd)
  if (threadIdx.x < TA) {
    const long long gi = rows[threadIdx.x];
    CQ[threadIdx.x] = gi >= 0 ? ebar[gi / md.N] : T(0);
    CP[threadIdx.x] = gi >= 0 ? T(1) : T(0);
  }
  T* gw = grad + md.off_w[t];
  for (int l = Lq - 1; l >= 0; l--) {
    const int in = md.in_of(t, l), out = md.width[l];
    if (l < Lq - 1 || stage == 2) lv = get_layer<T>(md, t, l, w, wsm, stage);  // else: the last layer is still staged
    __syncthreads();
    const T* ho = H + md.h_off(l) * TAP;
    const T* ado = AD + md.h_off(l) * TAP;
    T* dql = DQ + md.h_off(l) * TAP;
    T* dpl = DP + md.h_off(l) * TAP;
    for (int idx = threadIdx.x; idx < out * TA; idx += ML_THREADS) {
      const int o = (idx / TA) * TAP + (idx % TA);
      T qa, pa;
      if (l < Lq - 1) {
        const T hh = ho[o], d1 = T(1) - hh * hh;
        pa = CP[o] * d1;
        qa = CQ[o] * d1 + CP[o] * (T(-2) * hh * d1 * ado[o]);
      } else {
        pa = CP[o];
        qa = CQ[o];
      }
      dql[o] = qa;
      dpl[o] = pa;
    }
    __syncthreads();
    ML_TICK(1, 2)
    // weight gradient of this layer, summed over the block's atoms: 2 inputs x 2 outputs per thread,
    // atoms four at a time (the padded row stride keeps the 16-byte loads of consecutive rows conflict-free)
    const T* hin = (l == 0) ? X : H + md.h_off(l - 1) * TAP;
    const T* hdi = (l == 0) ? V : HD + md.h_off(l - 1) * TAP;
    const int woff = md.w_off(t, l);
    const int nj2 = (out + 1) >> 1, ni2 = (in + 1) >> 1;
    for (int tile = threadIdx.x; tile < nj2 * ni2; tile += ML_THREADS) {
      const int j0 = (tile % nj2) * 2, i0 = (tile / nj2) * 2;
      const int j1 = j0 + 1 < out ? j0 + 1 : j0, i1 = i0 + 1 < in ? i0 + 1 : i0;
      T g00 = T(0), g01 = T(0), g10 = T(0), g11 = T(0);
      auto dot4 = [](const T4 x, const T4 y) { return x.x * y.x + x.y * y.y + x.z * y.z + x.w * y.w; };
#pragma unroll 2
      for (int a = 0; a < TA; a += 4) {
        const T4 h0 = *reinterpret_cast<const T4*>(hin + i0 * TAP + a), h1 = *reinterpret_cast<const T4*>(hin + i1 * TAP + a);
        const T4 d0 = *reinterpret_cast<const T4*>(hdi + i0 * TAP + a), d1 = *reinterpret_cast<const T4*>(hdi + i1 * TAP + a);
        const T4 qa0 = *reinterpret_cast<const T4*>(dql + j0 * TAP + a), qa1 = *reinterpret_cast<const T4*>(dql + j1 * TAP + a);
        const T4 pa0 = *reinterpret_cast<const T4*>(dpl + j0 * TAP + a), pa1 = *reinterpret_cast<const T4*>(dpl + j1 * TAP + a);
        g00 += dot4(h0, qa0) + dot4(d0, pa0);
        g01 += dot4(h0, qa1) + dot4(d0, pa1);
        g10 += dot4(h1, qa0) + dot4(d1, pa0);
        g11 += dot4(h1, qa1) + dot4(d1, pa1);
      }
      atomicAdd(gw + woff + i0 * out + j0, g00);
      if (j0 + 1 < out) atomicAdd(gw + woff + i0 * out + j0 + 1, g01);
      if (i0 + 1 < in) {
        atomicAdd(gw + woff + i1 * out + j0, g10);
        if (j0 + 1 < out) atomicAdd(gw + woff + i1 * out + j0 + 1, g11);
      }
    }
    // bias gradient
    for (int j = threadIdx.x; j < out; j += ML_THREADS) {
      T g = T(0);
      for (int a = 0; a < TA; a++) g += dql[j * TAP + a];
      atomicAdd(gw + woff + in * out + j, g);
    }
    ML_TICK(1, 3)
    // cotangents on the layer input
    dense_bwd<T, TA>(in, out, lv, dql, CQ, dpl, CP);
    ML_TICK(1, 4)
  }
  // CQ = dS/dx, CP = dS/dv  ->  dL/dAF, kept in V for the contraction below
  for (int idx = threadIdx.x; idx < Fm * TA; idx += ML_THREADS) {
    const int i = idx % Fm, a = idx / Fm;
    const long long gi = rows[a];
    T g = T(0);
    if (gi >= 0 && i < F) {
      const T den = af[gi * Fm + i] + T(1e-3);
      g = CQ[i * TAP + a] / den + CP[i * TAP + a] * (-u[gi * Fm + i] / (den * den));
    }
    if (gi >= 0) gaf[gi * Fm + i] = g;
    if (i < F) V[i * TAP + a] = g;
  }
  for (int i = threadIdx.x; i < F; i += ML_THREADS) {
    T g = T(0);
    for (int a = 0; a < TA; a++) g -= CQ[i * TAP + a];
    atomicAdd(grad + md.off_mu[t] + i, g);
  }
  ML_TICK(1, 5)
  if (vrow) {
    __syncthreads();
    // dL/dalpha (fingerprint part) = sum_atoms dL/dAF[c(q)] * dAF[c(q)]/dalpha[q]; alpha2b and alpha3b
    // are contiguous in theta, q runs over both
    const int Fr = md.Fr[t], Fa = md.Fa[t], n2 = md.nt * Fr, nq = n2 + md.C * 3 * Fa;
    for (int q = threadIdx.x; q < nq; q += ML_THREADS) {
      const int ch = q < n2 ? (q % Fr) : Fr + ((q - n2) / 3) % Fa;
      // position of parameter q in the rows the fingerprint sweep wrote: its accumulator layout
      // alpha2b[nt,Frmax] | alpha3b[C,3*Famax] (equal to q when every species has the same channel counts)
      int qa;
      if (q < n2) qa = (q / Fr) * md.Frmax + (q % Fr);
      else {
        const int r = q - n2, sc = r / 3, s = sc / Fa;
        qa = md.nt * md.Frmax + (s * md.Famax + (sc - s * Fa)) * 3 + (r - sc * 3);
      }
      T g = T(0);
      for (int a = 0; a < TA; a++) {
        const long long gi = rows[a];
        if (gi >= 0) g += V[ch * TAP + a] * vrow[gi * nv + qa];
      }
      if (g != T(0)) atomicAdd(grad + md.off_a2[t] + q, g);
    }
  }
  ML_TICK(1, 6)
}
