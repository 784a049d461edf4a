// Per-species MLP energy head of the fused path (included by fused.cu inside namespace stafb).
//
// x = log(AF+1e-3) - mu ; Dense(tanh)... Dense(1)  (staf_models/staf_model.py:188-191,
// libstaf/src/mlp/staf_mlp_ort.cc:196-242 of the reference).
//
// The layers of this network are small (25-64-32-1 up to 60-140-140-1), so a block-wide product per layer spends
// its time in barriers.  Here every WARP carries AW atoms (4, 2 or 1) of one species through all layers on its own:
// its vectors live in a private slice of shared memory, feature-major ([feature][atom], one 16-byte row per
// feature at AW = 4), and only __syncwarp() separates the layers.  The eight warps of a block share the staged
// Dense layers (all layers at kernel start, one layer at a time - the only mode with block barriers between
// layers - or none, read from global memory).
//   forward   Y[j][a]  = sum_i W[i][j] X[i][a]   lane = output j (and j+32): one broadcast row load of X and two
//                                                conflict-free weight loads per 2*AW FMAs
//   backward  Xo[i][a] = sum_j W[i][j] D[j][a]   lane = input i: the lane's weight row 16 bytes at a time (row
//                                                stride = 4 mod 32 words: conflict-free), D rows broadcast
//   dL/dW     G[i][j]  = sum_a h[i][a] q[j][a]   needs every atom of the block: once all warps are through, the
//                                                block forms it 4 x 4 per thread over the eight warps' slices
#pragma once
#include <cuda_pipeline.h>

constexpr int ML_WARPS = ML_THREADS / 32;

// row stride of a staged layer with `out` columns: smallest value >= out that is 4 mod 32
__host__ __device__ inline int ml_ld(int out) { return ((out + 27) / 32) * 32 + 4; }

template <class T>
struct LayerView {
  const T* W;  // element (i,j) at W[i*ld + j]; columns out..ld-1 are zero
  const T* B;  // bias
  int ld;
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

template <class T>
__device__ __forceinline__ LayerView<T> layer_view(int in, int out, const T* base) {
  LayerView<T> v;
  v.ld = ml_ld(out);
  v.W = base; v.B = base + in * v.ld;
  return v;
}

// Dense layer l of species t; wp = the species' packed weights in global memory.  WG: the weights stay in global
// memory (the layers do not fit next to the warps' slices).  Otherwise stage 2: every layer was staged when the
// kernel started (wsm holds them back to back); stage 1: stage this layer now, between two block barriers - every
// warp of the block calls this at the same point.
template <class T, bool WG>
__device__ __forceinline__ LayerView<T> get_layer(const ModelDev& md, int t, int l, const T* __restrict__ wp, T* wsm,
                                                 int stage) {
  const int in = md.in_of(t, l), out = md.width[l];
  int off = 0;
  for (int k = 0; k < l; k++) off += ml_layer_words(md.in_of(t, k), md.width[k]);
  if (WG) return layer_view<T>(in, out, wp + off);
  if (stage == 2) return layer_view<T>(in, out, wsm + off);
  __syncthreads();  // every warp is done with the layer staged before
  stage_words<T>(wp + off, wsm, ml_layer_words(in, out));
  __pipeline_wait_prior(0);
  __syncthreads();
  return layer_view<T>(in, out, wsm);
}

// tanh for the activations: fp32 as 1 - 2/(2^(2x log2 e) + 1) with the hardware exponential and reciprocal
// (absolute error of a few 1e-7, saturates correctly at +-1), fp64 the library function
__device__ __forceinline__ float ml_tanh(float x) {
  const float e = ex2_fast(x * 2.885390081777927f);
  return 1.0f - __fdividef(2.0f, e + 1.0f);
}
__device__ __forceinline__ double ml_tanh(double x) { return tanh(x); }

// one [feature] row of a warp's slice: AW consecutive reals
template <class T, int AW> struct RowIO;
template <> struct RowIO<float, 4> {
  static __device__ __forceinline__ void ld(const float* p, float (&x)[4]) {
    const float4 v = *reinterpret_cast<const float4*>(p);
    x[0] = v.x; x[1] = v.y; x[2] = v.z; x[3] = v.w;
  }
  static __device__ __forceinline__ void st(float* p, const float (&x)[4]) {
    *reinterpret_cast<float4*>(p) = make_float4(x[0], x[1], x[2], x[3]);
  }
};
template <> struct RowIO<float, 2> {
  static __device__ __forceinline__ void ld(const float* p, float (&x)[2]) {
    const float2 v = *reinterpret_cast<const float2*>(p);
    x[0] = v.x; x[1] = v.y;
  }
  static __device__ __forceinline__ void st(float* p, const float (&x)[2]) {
    *reinterpret_cast<float2*>(p) = make_float2(x[0], x[1]);
  }
};
template <> struct RowIO<double, 4> {
  static __device__ __forceinline__ void ld(const double* p, double (&x)[4]) {
    const double2 a = *reinterpret_cast<const double2*>(p), b = *reinterpret_cast<const double2*>(p + 2);
    x[0] = a.x; x[1] = a.y; x[2] = b.x; x[3] = b.y;
  }
  static __device__ __forceinline__ void st(double* p, const double (&x)[4]) {
    *reinterpret_cast<double2*>(p) = make_double2(x[0], x[1]);
    *reinterpret_cast<double2*>(p + 2) = make_double2(x[2], x[3]);
  }
};
template <> struct RowIO<double, 2> {
  static __device__ __forceinline__ void ld(const double* p, double (&x)[2]) {
    const double2 a = *reinterpret_cast<const double2*>(p);
    x[0] = a.x; x[1] = a.y;
  }
  static __device__ __forceinline__ void st(double* p, const double (&x)[2]) {
    *reinterpret_cast<double2*>(p) = make_double2(x[0], x[1]);
  }
};
template <class T> struct RowIO<T, 1> {
  static __device__ __forceinline__ void ld(const T* p, T (&x)[1]) { x[0] = p[0]; }
  static __device__ __forceinline__ void st(T* p, const T (&x)[1]) { p[0] = x[0]; }
};
// four consecutive weights of a row (16-byte aligned)
__device__ __forceinline__ void ml_ld4(const float* p, float (&w)[4]) {
  const float4 v = *reinterpret_cast<const float4*>(p);
  w[0] = v.x; w[1] = v.y; w[2] = v.z; w[3] = v.w;
}
__device__ __forceinline__ void ml_ld4(const double* p, double (&w)[4]) {
  const double2 a = *reinterpret_cast<const double2*>(p), b = *reinterpret_cast<const double2*>(p + 2);
  w[0] = a.x; w[1] = a.y; w[2] = b.x; w[3] = b.y;
}

// four consecutive words of a gradient row in one atomic (fp32, 16-byte aligned address); fp64 has no such form
__device__ __forceinline__ void ml_add4(float* p, float a, float b, float c, float d) {
  atomicAdd(reinterpret_cast<float4*>(p), make_float4(a, b, c, d));
}
__device__ __forceinline__ void ml_add4(double* p, double a, double b, double c, double d) {
  atomicAdd(p, a); atomicAdd(p + 1, b); atomicAdd(p + 2, c); atomicAdd(p + 3, d);
}

// ---- dense products, two forms.  Narrow layers (at most 64 wide): two output columns or one weight row per lane.
// Y[j][a] = act( b[j] + sum_i X[i][a] W[i,j] ), one warp, AW atoms; a lane owns outputs j0+lane and j0+32+lane
// of every group of 64.  The caller separates this from the producer of X with __syncwarp().
template <class T, int AW, bool TANH, bool BIAS>
__device__ __forceinline__ void warp_dense_fwd_narrow(int in, int out, const LayerView<T> lv, const T* __restrict__ X,
                                               T* __restrict__ Y, int lane) {
  const int ld = lv.ld;
  for (int j0 = 0; j0 < out; j0 += 64) {
    const int ja = j0 + lane, jb = ja + 32;
    const bool two = j0 + 32 < out;  // warp-uniform
    // a lane past the last output reads the last column and drops the result
    const T* wa = lv.W + (ja < out ? ja : out - 1);
    const T* wb = lv.W + (jb < out ? jb : out - 1);
    T acc0[AW], acc1[AW];
#pragma unroll
    for (int a = 0; a < AW; a++) acc0[a] = acc1[a] = T(0);
    if (two) {
#pragma unroll 4
      for (int i = 0; i < in; i++) {
        T x[AW];
        RowIO<T, AW>::ld(X + i * AW, x);
        const T w0 = wa[i * ld], w1 = wb[i * ld];
#pragma unroll
        for (int a = 0; a < AW; a++) { acc0[a] += w0 * x[a]; acc1[a] += w1 * x[a]; }
      }
    } else {
#pragma unroll 4
      for (int i = 0; i < in; i++) {
        T x[AW];
        RowIO<T, AW>::ld(X + i * AW, x);
        const T w0 = wa[i * ld];
#pragma unroll
        for (int a = 0; a < AW; a++) acc0[a] += w0 * x[a];
      }
    }
    if (ja < out) {
      const T b = BIAS ? lv.B[ja] : T(0);
#pragma unroll
      for (int a = 0; a < AW; a++) { acc0[a] += b; if (TANH) acc0[a] = ml_tanh(acc0[a]); }
      RowIO<T, AW>::st(Y + ja * AW, acc0);
    }
    if (two && jb < out) {
      const T b = BIAS ? lv.B[jb] : T(0);
#pragma unroll
      for (int a = 0; a < AW; a++) { acc1[a] += b; if (TANH) acc1[a] = ml_tanh(acc1[a]); }
      RowIO<T, AW>::st(Y + jb * AW, acc1);
    }
  }
}

// Xo[i][a] = sum_j D[j][a] W[i,j]  (and the same for a second cotangent D2 -> Xo2 when TWO), one warp, AW atoms;
// a lane owns input i0+lane of every group of 32 and walks its weight row four columns at a time (pointers that
// advance by constants; summation order j = 0, 1, 2, ...).
template <class T, int AW, bool TWO>
__device__ __forceinline__ void warp_dense_bwd_narrow(int in, int out, const LayerView<T> lv, const T* __restrict__ D,
                                               T* __restrict__ Xo, const T* __restrict__ D2, T* __restrict__ Xo2,
                                               int lane) {
  const int ld = lv.ld;
  for (int i0 = 0; i0 < in; i0 += 32) {
    const int i = i0 + lane;
    const T* wr = lv.W + (size_t)(i < in ? i : in - 1) * ld;  // a lane past the last input repeats the last row
    const T* pd = D;
    const T* pd2 = TWO ? D2 : D;
    T acc[AW], acc2[AW];
#pragma unroll
    for (int a = 0; a < AW; a++) acc[a] = acc2[a] = T(0);
#pragma unroll 2
    for (int n = out >> 2; n > 0; n--) {
      T w[4];
      ml_ld4(wr, w);
#pragma unroll
      for (int r = 0; r < 4; r++) {
        T d[AW];
        RowIO<T, AW>::ld(pd + r * AW, d);
#pragma unroll
        for (int a = 0; a < AW; a++) acc[a] += w[r] * d[a];
        if (TWO) {
          RowIO<T, AW>::ld(pd2 + r * AW, d);
#pragma unroll
          for (int a = 0; a < AW; a++) acc2[a] += w[r] * d[a];
        }
      }
      wr += 4; pd += 4 * AW; pd2 += 4 * AW;
    }
    for (int n = out & 3; n > 0; n--) {
      const T w = wr[0];
      T d[AW];
      RowIO<T, AW>::ld(pd, d);
#pragma unroll
      for (int a = 0; a < AW; a++) acc[a] += w * d[a];
      if (TWO) {
        RowIO<T, AW>::ld(pd2, d);
#pragma unroll
        for (int a = 0; a < AW; a++) acc2[a] += w * d[a];
      }
      wr++; pd += AW; pd2 += AW;
    }
    if (i < in) {
      RowIO<T, AW>::st(Xo + i * AW, acc);
      if (TWO) RowIO<T, AW>::st(Xo2 + i * AW, acc2);
    }
  }
}

// ---- wide layers: up to four output columns or two weight rows per lane
// NG output columns per lane (j, j+32, ...): acc[g][a] += sum_i X[i][a] W[i, j + 32 g].  One broadcast row load of X
// serves NG * AW multiply-adds and the NG sums are independent chains.
template <class T, int AW, int NG>
__device__ __forceinline__ void ml_fwd_cols(int in, int ld, const T* __restrict__ w0, const T* __restrict__ w1,
                                            const T* __restrict__ w2, const T* __restrict__ w3,
                                            const T* __restrict__ X, T (&acc)[4][AW]) {
#pragma unroll 4
  for (int i = 0; i < in; i++) {
    T x[AW];
    RowIO<T, AW>::ld(X + i * AW, x);
    const T v0 = w0[i * ld], v1 = NG > 1 ? w1[i * ld] : T(0), v2 = NG > 2 ? w2[i * ld] : T(0),
            v3 = NG > 3 ? w3[i * ld] : T(0);
#pragma unroll
    for (int a = 0; a < AW; a++) {
      acc[0][a] += v0 * x[a];
      if (NG > 1) acc[1][a] += v1 * x[a];
      if (NG > 2) acc[2][a] += v2 * x[a];
      if (NG > 3) acc[3][a] += v3 * x[a];
    }
  }
}

// Y[j][a] = act( b[j] + sum_i X[i][a] W[i,j] ), one warp, AW atoms; a lane owns outputs j0+lane, j0+32+lane, ... of
// every group of 128 (as many of the four as the layer has).  The caller separates this from the producer of X
// with __syncwarp().
template <class T, int AW, bool TANH, bool BIAS>
__device__ __forceinline__ void warp_dense_fwd_wide(int in, int out, const LayerView<T> lv, const T* __restrict__ X,
                                               T* __restrict__ Y, int lane) {
  const int ld = lv.ld;
  for (int j0 = 0; j0 < out; j0 += 128) {
    const int ng = (out - j0 + 31) >> 5;  // 32-column groups left; warp-uniform
    // a lane past the last output reads the last column and drops the result
    T acc[4][AW];
#pragma unroll
    for (int g = 0; g < 4; g++)
#pragma unroll
      for (int a = 0; a < AW; a++) acc[g][a] = T(0);
    const int last = out - 1, jl = j0 + lane;
    const T* w0 = lv.W + (jl < out ? jl : last);
    const T* w1 = lv.W + (jl + 32 < out ? jl + 32 : last);
    const T* w2 = lv.W + (jl + 64 < out ? jl + 64 : last);
    const T* w3 = lv.W + (jl + 96 < out ? jl + 96 : last);
    if (ng >= 4) ml_fwd_cols<T, AW, 4>(in, ld, w0, w1, w2, w3, X, acc);
    else if (ng == 3) ml_fwd_cols<T, AW, 3>(in, ld, w0, w1, w2, w3, X, acc);
    else if (ng == 2) ml_fwd_cols<T, AW, 2>(in, ld, w0, w1, w2, w3, X, acc);
    else ml_fwd_cols<T, AW, 1>(in, ld, w0, w1, w2, w3, X, acc);
#pragma unroll
    for (int g = 0; g < 4; g++) {
      const int j = j0 + 32 * g + lane;
      if (g < ng && j < out) {
        const T b = BIAS ? lv.B[j] : T(0);
#pragma unroll
        for (int a = 0; a < AW; a++) { acc[g][a] += b; if (TANH) acc[g][a] = ml_tanh(acc[g][a]); }
        RowIO<T, AW>::st(Y + j * AW, acc[g]);
      }
    }
  }
}

// NR weight rows per lane (i, i+32): acc[r][a] += sum_j D[j][a] W[i + 32 r, j] (and acc2 with D2 when TWO), four
// columns per trip, pointers that advance by constants; summation order j = 0, 1, 2, ...  The D rows are loaded
// once for both weight rows.
template <class T, int AW, bool TWO, int NR>
__device__ __forceinline__ void ml_bwd_rows(int out, const T* __restrict__ wr0, const T* __restrict__ wr1,
                                            const T* __restrict__ D, const T* __restrict__ D2, T (&acc)[2][AW],
                                            T (&acc2)[2][AW]) {
  const T* pd = D;
  const T* pd2 = TWO ? D2 : D;
#pragma unroll 2
  for (int n = out >> 2; n > 0; n--) {
    T w[2][4];
    ml_ld4(wr0, w[0]);
    if (NR == 2) ml_ld4(wr1, w[1]);
#pragma unroll
    for (int r = 0; r < 4; r++) {
      T d[AW];
      RowIO<T, AW>::ld(pd + r * AW, d);
#pragma unroll
      for (int q = 0; q < NR; q++)
#pragma unroll
        for (int a = 0; a < AW; a++) acc[q][a] += w[q][r] * d[a];
      if (TWO) {
        RowIO<T, AW>::ld(pd2 + r * AW, d);
#pragma unroll
        for (int q = 0; q < NR; q++)
#pragma unroll
          for (int a = 0; a < AW; a++) acc2[q][a] += w[q][r] * d[a];
      }
    }
    wr0 += 4; wr1 += 4; pd += 4 * AW; pd2 += 4 * AW;
  }
  for (int n = out & 3; n > 0; n--) {
    T w[2];
    w[0] = wr0[0];
    w[1] = NR == 2 ? wr1[0] : T(0);
    T d[AW];
    RowIO<T, AW>::ld(pd, d);
#pragma unroll
    for (int q = 0; q < NR; q++)
#pragma unroll
      for (int a = 0; a < AW; a++) acc[q][a] += w[q] * d[a];
    if (TWO) {
      RowIO<T, AW>::ld(pd2, d);
#pragma unroll
      for (int q = 0; q < NR; q++)
#pragma unroll
        for (int a = 0; a < AW; a++) acc2[q][a] += w[q] * d[a];
    }
    wr0++; wr1++; pd += AW; pd2 += AW;
  }
}

// Xo[i][a] = sum_j D[j][a] W[i,j]  (and the same for a second cotangent D2 -> Xo2 when TWO), one warp, AW atoms;
// a lane owns inputs i0+lane and i0+32+lane of every group of 64 and walks their weight rows four columns at a time.
template <class T, int AW, bool TWO>
__device__ __forceinline__ void warp_dense_bwd_wide(int in, int out, const LayerView<T> lv, const T* __restrict__ D,
                                               T* __restrict__ Xo, const T* __restrict__ D2, T* __restrict__ Xo2,
                                               int lane) {
  const int ld = lv.ld;
  for (int i0 = 0; i0 < in; i0 += 64) {
    const int ia = i0 + lane, ib = ia + 32;
    const bool two = i0 + 32 < in;  // warp-uniform
    // a lane past the last input repeats the last row and drops the result
    const T* wra = lv.W + (size_t)(ia < in ? ia : in - 1) * ld;
    const T* wrb = lv.W + (size_t)(ib < in ? ib : in - 1) * ld;
    T acc[2][AW], acc2[2][AW];
#pragma unroll
    for (int a = 0; a < AW; a++) acc[0][a] = acc[1][a] = acc2[0][a] = acc2[1][a] = T(0);
    if (two) ml_bwd_rows<T, AW, TWO, 2>(out, wra, wrb, D, D2, acc, acc2);
    else ml_bwd_rows<T, AW, TWO, 1>(out, wra, wrb, D, D2, acc, acc2);
    if (ia < in) {
      RowIO<T, AW>::st(Xo + ia * AW, acc[0]);
      if (TWO) RowIO<T, AW>::st(Xo2 + ia * AW, acc2[0]);
    }
    if (two && ib < in) {
      RowIO<T, AW>::st(Xo + ib * AW, acc[1]);
      if (TWO) RowIO<T, AW>::st(Xo2 + ib * AW, acc2[1]);
    }
  }
}

// The form is a template parameter of the kernels, chosen per model by the widest layer: the wide form shares every
// operand load between more multiply-adds and keeps more independent sums in flight, which pays for 140-wide layers
// (-9 % / -5 % on the 60-140-140-1 kernels) and costs about a microsecond on 64-wide ones.
template <class T, int AW, bool TANH, bool BIAS, bool WIDE>
__device__ __forceinline__ void warp_dense_fwd(int in, int out, const LayerView<T> lv, const T* __restrict__ X,
                                               T* __restrict__ Y, int lane) {
  if (WIDE) warp_dense_fwd_wide<T, AW, TANH, BIAS>(in, out, lv, X, Y, lane);
  else warp_dense_fwd_narrow<T, AW, TANH, BIAS>(in, out, lv, X, Y, lane);
}
template <class T, int AW, bool TWO, bool WIDE>
__device__ __forceinline__ void warp_dense_bwd(int in, int out, const LayerView<T> lv, const T* __restrict__ D,
                                               T* __restrict__ Xo, const T* __restrict__ D2, T* __restrict__ Xo2,
                                               int lane) {
  if (WIDE) warp_dense_bwd_wide<T, AW, TWO>(in, out, lv, D, Xo, D2, Xo2, lane);
  else warp_dense_bwd_narrow<T, AW, TWO>(in, out, lv, D, Xo, D2, Xo2, lane);
}

// global row of atom slot a of this block (species t, first species-local index q0), or -1 past the end
__device__ __forceinline__ long long ml_atom_row(const ModelDev& md, int t, int q0, int nat, int a) {
  const int q = q0 + a;
  if (q >= nat) return -1;
  const int b = q / md.tipos[t];
  return (long long)b * md.N + md.shift[t] + (q - b * md.tipos[t]);
}

// words of a warp's slice in the two kernels
__host__ __device__ inline size_t ml_fwd_words(int Fm, int Hs, int mw, int AW) {
  return (size_t)(Fm + Hs + 2 * mw) * AW;
}
__host__ __device__ inline size_t ml_bwd_words(int Fm, int Hs, int mw, int AW) {
  return (size_t)(2 * Fm + 5 * Hs + 4 * mw) * AW;
}

// Forward: e_i, the activations for the backward kernel and netderiv = d(sum e)/dAF.
// acts: [block][warp][Hs][AW], the warps' activation slices as they are.
template <class T, int AW, bool WG, bool WIDE>
__global__ void __launch_bounds__(ML_THREADS)
    k_mlp_fwd(ModelDev md, int nf, const T* __restrict__ theta, const T* __restrict__ wpack, int wstride,
              const T* __restrict__ af, T* __restrict__ acts, T* __restrict__ e_atom, T* __restrict__ netderiv,
              int stage, int wsm_words) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  constexpr int TB = ML_WARPS * AW;
  int t, q0;
  locate_block(md, nf, TB, t, q0);
  const int nat = nf * md.tipos[t];
  const int F = md.Fr[t] + md.Fa[t], Lq = md.n_dense, Fm = md.Fmax, Hs = md.Hsum, mw = md.maxw;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  T* wsm = reinterpret_cast<T*>(smem_raw);  // staged layer(s)
  T* X = wsm + wsm_words + (size_t)warp * ml_fwd_words(Fm, Hs, mw, AW);  // [Fm][AW]
  T* H = X + Fm * AW;                                                    // [Hs][AW]
  T* C0 = H + Hs * AW;                                                   // [mw][AW]
  T* C1 = C0 + mw * AW;                                                  // [mw][AW]
  const T* mu = theta + md.off_mu[t];
  const T* w = wpack + (size_t)t * wstride;  // this species' packed layers
  long long gi[AW];
#pragma unroll
  for (int a = 0; a < AW; a++) gi[a] = ml_atom_row(md, t, q0, nat, warp * AW + a);
  if (!WG && stage == 2) {
    int words = 0;
    for (int l = 0; l < Lq; l++) words += ml_layer_words(md.in_of(t, l), md.width[l]);
    stage_words<T>(w, wsm, words);
  }
  chain_wait();  // the packed weights are older than the preceding kernel; everything read below is its output
  // lanes on consecutive fingerprints of one atom
#pragma unroll
  for (int a = 0; a < AW; a++)
    for (int i = lane; i < F; i += 32)
      X[i * AW + a] = gi[a] >= 0 ? r_log(af[gi[a] * Fm + i] + T(1e-3)) - mu[i] : T(0);
  if (!WG && stage == 2) {
    __pipeline_wait_prior(0);
    __syncthreads();
  }
  const T* hin = X;
  LayerView<T> lv;
  for (int l = 0; l < Lq; l++) {
    const int in = md.in_of(t, l), out = md.width[l];
    lv = get_layer<T, WG>(md, t, l, w, wsm, stage);
    __syncwarp();
    T* hout = H + md.h_off(l) * AW;
    if (l < Lq - 1) warp_dense_fwd<T, AW, true, true, WIDE>(in, out, lv, hin, hout, lane);
    else warp_dense_fwd<T, AW, false, true, WIDE>(in, out, lv, hin, hout, lane);
    hin = hout;
  }
  __syncwarp();
  // activations: the warp's slice as it is
  T* ab = acts + ((size_t)blockIdx.x * ML_WARPS + warp) * Hs * AW;
  for (int idx = lane; idx < Hs * AW; idx += 32) ab[idx] = H[idx];
  if (lane < AW && gi[0] >= 0) {
    long long g = gi[0];
#pragma unroll
    for (int a = 1; a < AW; a++)
      if (lane == a) g = gi[a];
    if (g >= 0) e_atom[g] = H[md.h_off(Lq - 1) * AW + lane];  // the loss kernel sums them per frame
  }
  // de/dx by the reverse sweep: cn = cotangent on the output of layer l
  T* cn = C0;
  T* cp = C1;
  if (lane < AW) cn[lane] = T(1);
  for (int l = Lq - 1; l >= 0; l--) {
    const int in = md.in_of(t, l), out = md.width[l];
    if (l < Lq - 1 || WG || stage == 2) lv = get_layer<T, WG>(md, t, l, w, wsm, stage);  // else: still staged
    __syncwarp();
    if (l < Lq - 1) {
      const T* hl = H + md.h_off(l) * AW;
      for (int idx = lane; idx < out * AW; idx += 32) cn[idx] *= (T(1) - hl[idx] * hl[idx]);
      __syncwarp();
    }
    warp_dense_bwd<T, AW, false, WIDE>(in, out, lv, cn, cp, nullptr, nullptr, lane);
    T* tmp = cn; cn = cp; cp = tmp;
  }
  __syncwarp();
#pragma unroll
  for (int a = 0; a < AW; a++) {
    if (gi[a] < 0) continue;
    for (int i = lane; i < Fm; i += 32)
      netderiv[gi[a] * Fm + i] = (i < F) ? cn[i * AW + a] / (af[gi[a] * Fm + i] + T(1e-3)) : T(0);
  }
}

// Backward of  S = sum_a ebar[a]*e[a] + sum_{a,c} u[a,c]*netderiv[a,c]  with respect to the
// weights, mu and AF: the first term is plain back-propagation, the second is the derivative
// of a directional derivative (tangent v = u/(AF+eps) pushed forward, then reversed) - what
// TensorFlow's autodiff does through grad_ene for the force loss (staf_model.py:191,225-228).
// The kernel also contracts dL/dAF with the per-atom d(AF)/d(alpha) rows left by the AF sweep
// (vrow), which yields the fingerprint part of dL/dalpha without another sweep over the triplets.
// fp32 with up to 2 atoms per warp: three blocks per SM fit by shared memory, so the registers are capped for three
template <class T, int AW, bool WG, bool WIDE>
__global__ void __launch_bounds__(ML_THREADS, (sizeof(T) == 4 && AW <= 2) ? 3 : 1)
    k_mlp_bwd(ModelDev md, int nf, const T* __restrict__ theta, const T* __restrict__ wpack, int wstride,
              const T* __restrict__ af, const T* __restrict__ acts, const T* __restrict__ ebar /*[nf]*/, const T* __restrict__ u /*[nf,N,Fmax]*/,
              const T* __restrict__ vrow /*[nf,N,nv] or null*/, int nv, T* __restrict__ gaf, T* __restrict__ grad,
              int stage, int wsm_words) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  constexpr int TB = ML_WARPS * AW;
  __shared__ long long rows[TB];
  int t, q0;
  locate_block(md, nf, TB, t, q0);
  const int nat = nf * md.tipos[t];
  const int F = md.Fr[t] + md.Fa[t], Lq = md.n_dense, Fm = md.Fmax, Hs = md.Hsum, mw = md.maxw;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const size_t slice = ml_bwd_words(Fm, Hs, mw, AW);
  T* wsm = reinterpret_cast<T*>(smem_raw);  // staged layer(s)
  T* base = wsm + wsm_words;
  // offsets inside a warp's slice
  const int oX = 0, oV = Fm * AW, oH = 2 * Fm * AW, oHD = oH + Hs * AW, oAD = oHD + Hs * AW, oDQ = oAD + Hs * AW,
            oDP = oDQ + Hs * AW, oC = oDP + Hs * AW;  // then four [mw][AW] cotangent buffers
  T* my = base + (size_t)warp * slice;
  T* X = my + oX;    // x
  T* V = my + oV;    // tangent on x
  T* H = my + oH;    // activations
  T* HD = my + oHD;  // tangents of the activations
  T* AD = my + oAD;  // tangents of the pre-activations
  T* DQ = my + oDQ;  // cotangents on the pre-activations, every layer (first-order channel)
  T* DP = my + oDP;  // cotangents on the tangents of the pre-activations
  const T* mu = theta + md.off_mu[t];
  const T* w = wpack + (size_t)t * wstride;  // this species' packed layers
  long long gi[AW];
#pragma unroll
  for (int a = 0; a < AW; a++) gi[a] = ml_atom_row(md, t, q0, nat, warp * AW + a);
  if (threadIdx.x < TB) rows[threadIdx.x] = ml_atom_row(md, t, q0, nat, threadIdx.x);
  if (!WG && stage == 2) {
    int words = 0;
    for (int l = 0; l < Lq; l++) words += ml_layer_words(md.in_of(t, l), md.width[l]);
    stage_words<T>(w, wsm, words);
  }
  chain_wait();  // the packed weights are older than the preceding kernel; everything read below is its output
#pragma unroll
  for (int a = 0; a < AW; a++) {
    for (int i = lane; i < F; i += 32) {
      T xv = T(0), vv = T(0);
      if (gi[a] >= 0) {
        const T den = af[gi[a] * Fm + i] + T(1e-3);
        xv = r_log(den) - mu[i];
        vv = u[gi[a] * Fm + i] / den;
      }
      X[i * AW + a] = xv;
      V[i * AW + a] = vv;
    }
  }
  {
    const T* ab = acts + ((size_t)blockIdx.x * ML_WARPS + warp) * Hs * AW;
    for (int idx = lane; idx < Hs * AW; idx += 32) {
      long long g = gi[0];
#pragma unroll
      for (int a = 1; a < AW; a++)
        if ((idx % AW) == a) g = gi[a];
      H[idx] = g >= 0 ? ab[idx] : T(0);
    }
  }
  if (!WG && stage == 2) {
    __pipeline_wait_prior(0);
    __syncthreads();
  }
  // forward tangent: AD = HDin W ; HD = AD * act'
  const T* hdin = V;
  LayerView<T> lv;
  for (int l = 0; l < Lq; l++) {
    const int in = md.in_of(t, l), out = md.width[l];
    lv = get_layer<T, WG>(md, t, l, w, wsm, stage);
    __syncwarp();
    T* ado = AD + md.h_off(l) * AW;
    T* hdo = HD + md.h_off(l) * AW;
    warp_dense_fwd<T, AW, false, false, WIDE>(in, out, lv, hdin, ado, lane);
    __syncwarp();
    const T* ho = H + md.h_off(l) * AW;
    for (int idx = lane; idx < out * AW; idx += 32)
      hdo[idx] = (l < Lq - 1) ? ado[idx] * (T(1) - ho[idx] * ho[idx]) : ado[idx];
    hdin = hdo;
  }
  __syncwarp();
  // reverse over (h, hd): (CQ, CP) = cotangents on (h, hd) of the current layer's output
  T* CQ = my + oC;
  T* CP = CQ + mw * AW;
  T* CQn = CP + mw * AW;
  T* CPn = CQn + mw * AW;
  if (lane < AW) {
    long long g = gi[0];
#pragma unroll
    for (int a = 1; a < AW; a++)
      if (lane == a) g = gi[a];
    CQ[lane] = g >= 0 ? ebar[g / md.N] : T(0);
    CP[lane] = g >= 0 ? T(1) : T(0);
  }
  for (int l = Lq - 1; l >= 0; l--) {
    const int in = md.in_of(t, l), out = md.width[l];
    if (l < Lq - 1 || WG || stage == 2) lv = get_layer<T, WG>(md, t, l, w, wsm, stage);  // else: still staged
    __syncwarp();
    const int ho_ = md.h_off(l) * AW;
    const T* ho = H + ho_;
    const T* ado = AD + ho_;
    T* dql = DQ + ho_;
    T* dpl = DP + ho_;
    for (int idx = lane; idx < out * AW; idx += 32) {
      T qa, pa;
      if (l < Lq - 1) {
        const T hh = ho[idx], d1 = T(1) - hh * hh;
        pa = CP[idx] * d1;
        qa = CQ[idx] * d1 + CP[idx] * (T(-2) * hh * d1 * ado[idx]);
      } else {
        pa = CP[idx];
        qa = CQ[idx];
      }
      dql[idx] = qa;
      dpl[idx] = pa;
    }
    __syncwarp();
    warp_dense_bwd<T, AW, true, WIDE>(in, out, lv, dql, CQn, dpl, CPn, lane);
    T* tq = CQ; CQ = CQn; CQn = tq;
    T* tp = CP; CP = CPn; CPn = tp;
  }
  __syncwarp();
  // CQ = dS/dx, CP = dS/dv  ->  dL/dAF, also kept in the free cotangent buffer G for the contraction below
  T* G = CQn;
#pragma unroll
  for (int a = 0; a < AW; a++) {
    for (int i = lane; i < Fm; i += 32) {
      T g = T(0);
      if (gi[a] >= 0 && i < F) {
        const T den = af[gi[a] * Fm + i] + T(1e-3);
        g = CQ[i * AW + a] / den + CP[i * AW + a] * (-u[gi[a] * Fm + i] / (den * den));
      }
      if (gi[a] >= 0) gaf[gi[a] * Fm + i] = g;
      G[i * AW + a] = g;
    }
  }
  const int oCQ = (int)(CQ - my), oG = (int)(G - my);  // the same in every warp (same number of swaps)
  __syncthreads();
  // ---- block-wide sums over the atoms of all warps
  T* gw = grad + md.off_w[t];
  // weight gradients of ALL layers in one pass: the 4 x 4 tiles (4 inputs x 4 outputs) of every layer are
  // numbered consecutively and dealt to the threads, so that the small layers do not leave most of the block
  // idle (rows past the end of a layer's last tile repeat its last row and are not written)
  // fp32, layer width a multiple of 4: the column tiles of a layer are shifted left by csh columns so that every
  // tile row starts on a 16-byte boundary of the gradient array and goes out as ONE 4-wide atomic add (the first
  // and the last tile of a row then hang over the edge and use scalar adds for the columns they have)
  int tile_end[STAFB_MAX_DENSE], csh[STAFB_MAX_DENSE];
  {
    int tot = 0;
    for (int l = 0; l < STAFB_MAX_DENSE; l++) {
      csh[l] = 0;
      if (l < Lq) {
        if (sizeof(T) == 4 && (md.width[l] & 3) == 0)
          csh[l] = (int)((reinterpret_cast<size_t>(gw + md.w_off(t, l)) >> 2) & 3);
        tot += ((md.in_of(t, l) + 3) >> 2) * ((md.width[l] + csh[l] + 3) >> 2);
      }
      tile_end[l] = tot;
    }
  }
  for (int tile = threadIdx.x; tile < tile_end[STAFB_MAX_DENSE - 1]; tile += ML_THREADS) {
    int l = 0;
#pragma unroll
    for (int q = 0; q < STAFB_MAX_DENSE - 1; q++) l += (tile >= tile_end[q]) ? 1 : 0;
    int tbeg = 0, sh = csh[0];
#pragma unroll
    for (int q = 0; q < STAFB_MAX_DENSE - 1; q++)
      if (q < l) { tbeg = tile_end[q]; sh = csh[q + 1]; }
    const int in = md.in_of(t, l), out = md.width[l];
    const int oin = (l == 0) ? oX : oH + md.h_off(l - 1) * AW;
    const int odi = (l == 0) ? oV : oHD + md.h_off(l - 1) * AW;
    const int oq = oDQ + md.h_off(l) * AW, op = oDP + md.h_off(l) * AW;
    const int woff = md.w_off(t, l);
    const int nj4 = (out + sh + 3) >> 2;
    const int lt = tile - tbeg, itl = lt / nj4, jt = lt - itl * nj4;
    const int j0 = (jt << 2) - sh, i0 = itl << 2;
    T g[16];
#pragma unroll
    for (int q = 0; q < 16; q++) g[q] = T(0);
    int ir[4], jr[4];
#pragma unroll
    for (int r = 0; r < 4; r++) {
      ir[r] = (i0 + r < in ? i0 + r : in - 1) * AW;
      jr[r] = (j0 + r < 0 ? 0 : (j0 + r < out ? j0 + r : out - 1)) * AW;
    }
#pragma unroll 2
    for (int wv = 0; wv < ML_WARPS; wv++) {
      const T* sb = base + (size_t)wv * slice;
      T hv[4][AW], dv[4][AW];
#pragma unroll
      for (int r = 0; r < 4; r++) {
        RowIO<T, AW>::ld(sb + oin + ir[r], hv[r]);
        RowIO<T, AW>::ld(sb + odi + ir[r], dv[r]);
      }
#pragma unroll
      for (int c = 0; c < 4; c++) {
        T qv[AW], pv[AW];
        RowIO<T, AW>::ld(sb + oq + jr[c], qv);
        RowIO<T, AW>::ld(sb + op + jr[c], pv);
#pragma unroll
        for (int r = 0; r < 4; r++)
#pragma unroll
          for (int a = 0; a < AW; a++) {
            g[4 * r + c] += hv[r][a] * qv[a];
            g[4 * r + c] += dv[r][a] * pv[a];
          }
      }
    }
    const bool whole = sizeof(T) == 4 && (out & 3) == 0 && j0 >= 0 && j0 + 4 <= out;  // aligned by construction
#pragma unroll
    for (int r = 0; r < 4; r++) {
      if (i0 + r >= in) continue;
      T* dst = gw + woff + (i0 + r) * out + j0;
      if (whole) {
        ml_add4(dst, g[4 * r], g[4 * r + 1], g[4 * r + 2], g[4 * r + 3]);
      } else {
#pragma unroll
        for (int c = 0; c < 4; c++)
          if (j0 + c >= 0 && j0 + c < out) atomicAdd(dst + c, g[4 * r + c]);
      }
    }
  }
  // bias gradients: the outputs of all layers in one pass (the DQ rows of the layers lie back to back)
  for (int jj = threadIdx.x; jj < Hs; jj += ML_THREADS) {
    int l = 0;
    while (l < Lq - 1 && jj >= md.h_off(l + 1)) l++;
    const int in = md.in_of(t, l), out = md.width[l], j = jj - md.h_off(l);
    T g = T(0);
#pragma unroll
    for (int wv = 0; wv < ML_WARPS; wv++) {
      const T* q = base + (size_t)wv * slice + oDQ + jj * AW;
#pragma unroll
      for (int a = 0; a < AW; a++) g += q[a];
    }
    atomicAdd(gw + md.w_off(t, l) + in * out + j, g);
  }
  for (int i = threadIdx.x; i < F; i += ML_THREADS) {
    T g = T(0);
    for (int wv = 0; wv < ML_WARPS; wv++) {
      const T* q = base + (size_t)wv * slice + oCQ + i * AW;
#pragma unroll
      for (int a = 0; a < AW; a++) g -= q[a];
    }
    atomicAdd(grad + md.off_mu[t] + i, g);
  }
  if (vrow) {
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
      for (int wv = 0; wv < ML_WARPS; wv++) {
        const T* gs = base + (size_t)wv * slice + oG + ch * AW;
#pragma unroll
        for (int a = 0; a < AW; a++) {
          const long long r = rows[wv * AW + a];
          if (r >= 0) g += gs[a] * vrow[r * nv + qa];
        }
      }
      if (g != T(0)) atomicAdd(grad + md.off_a2[t] + q, g);
    }
  }
}
