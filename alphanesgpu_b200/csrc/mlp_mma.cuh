// fp32 MLP energy head on the tensor cores (included by fused.cu inside namespace stafb, after mlp.cuh): the
// opt-in arm of the MLP kernels (STAFB_MLP_MMA=1 when the model is created).
//
// Same mathematics as k_mlp_fwd / k_mlp_bwd of mlp.cuh (staf_models/staf_model.py:188-195,225-228 of the
// reference).  Those kernels issue one FMA per multiply-add plus the shared-memory loads that feed it; here every
// dense product runs as mma.sync.m16n8k8 (TF32 operands, fp32 accumulation) on tiles of 16 atoms, with both
// operands split into a TF32 head and a TF32 remainder and three products per tile (x_lo*w_hi + x_hi*w_lo +
// x_hi*w_hi), which keeps the result at fp32 accuracy (the dropped lo*lo term is 2^-22 relative; errors against
// fp64 on the 60-140-140-1 model equal those of the FMA kernels).  Instructions per atom fall threefold, but on
// B200 this instruction issues at about one per 30 cycles per SM (and about 180 cycles apart within one warp),
// so the kernels end up 1.4-2x slower than the FMA kernels: 22 / 46 us against 16 / 31 us (forward / backward,
// 3072 atoms, 25-64-32-1), 79 against 42 us forward at 24,576 atoms.  That is why the FMA kernels stay the default.
//
// A block carries 16 atoms of one species through all layers; its vectors are rows of shared-memory buffers
// [16][ld] with ld = 4 mod 32 words, so that the A fragments (row = atom, column = feature) load without bank
// conflicts, and its warps (four by default) share every product by output tiles, with a block barrier between
// layers.  The Dense layers come pre-split and pre-ordered by fragment (k_prep, mm_pack_value below): per 8 x 8
// tile one 16-byte word per lane {hi(b0), hi(b1), lo(b0), lo(b1)}, once for the forward use (k = input,
// n = output) and once for the reverse use (k = output, n = input).  Every block needs every fragment exactly
// once, so they are not staged in shared memory: each warp streams its tiles' fragments from global memory (L2)
// through a small ring of registers, several k-steps ahead of their use.  The weight gradients of the block's 16
// atoms are formed by the same instruction ((feature x output) tiles dealt to the warps) and added to the
// gradient with atomics.
#pragma once

constexpr int MM_ATOMS = 16;  // atoms per block: the rows of one MMA tile
constexpr int MM_MAX_WARPS = 8;

__host__ __device__ inline int mm_pad8(int x) { return (x + 7) & ~7; }
// row stride of a [16][cols] buffer: the smallest value >= cols that is 4 mod 32
__host__ __device__ inline int mm_ld(int cols) { return ((cols + 27) / 32) * 32 + 4; }
// packed words of one Dense layer: forward fragments, reverse fragments, bias (padded to the tile width)
__host__ __device__ inline int mm_layer_words(int in, int out) {
  return 4 * mm_pad8(in) * mm_pad8(out) + mm_pad8(out);
}

struct MmShape {
  int L, F, Fp;                    // layers, fingerprints of this species, padded
  int in[STAFB_MAX_DENSE], out[STAFB_MAX_DENSE];
  int hoff[STAFB_MAX_DENSE + 1];   // column of layer l's output in an activation row (padded widths)
  int woff[STAFB_MAX_DENSE + 1];   // word offset of layer l in the species' pack
  int ldx, ldh, ldc;
};

__host__ __device__ inline MmShape mm_shape(const ModelDev& md, int t) {
  MmShape s;
  s.L = md.n_dense;
  s.F = md.Fr[t] + md.Fa[t];
  s.Fp = mm_pad8(md.Fmax);
  s.hoff[0] = 0; s.woff[0] = 0;
  int mw = s.Fp;
  for (int l = 0; l < STAFB_MAX_DENSE; l++) {
    const bool on = l < md.n_dense;
    s.in[l] = on ? md.in_of(t, l) : 0;
    s.out[l] = on ? md.width[l] : 0;
    s.hoff[l + 1] = s.hoff[l] + (on ? mm_pad8(md.width[l]) : 0);
    s.woff[l + 1] = s.woff[l] + (on ? mm_layer_words(s.in[l], s.out[l]) : 0);
    if (on && mm_pad8(md.width[l]) > mw) mw = mm_pad8(md.width[l]);
  }
  s.ldx = mm_ld(s.Fp + 8);
  s.ldh = mm_ld(s.hoff[md.n_dense] + 8);  // the weight-gradient tiles read up to 8 columns past a layer's rows
  s.ldc = mm_ld(mw);
  return s;
}
// words of the largest pack over the species (the stride between two species' packs)
static inline size_t mm_pack_words(const ModelDev& md) {
  size_t best = 0;
  for (int t = 0; t < md.nt; t++) {
    const MmShape s = mm_shape(md, t);
    best = (size_t)s.woff[md.n_dense] > best ? (size_t)s.woff[md.n_dense] : best;
  }
  return best;
}
// shared-memory words of a block in the two kernels
static inline size_t mm_fwd_words(const ModelDev& md) {
  const MmShape s = mm_shape(md, 0);  // the strides depend on Fmax and the widths only
  return (size_t)MM_ATOMS * (s.ldx + s.ldh + 2 * s.ldc);
}
static inline size_t mm_bwd_words(const ModelDev& md) {
  const MmShape s = mm_shape(md, 0);
  return (size_t)MM_ATOMS * (4 * s.ldx + 4 * s.ldh);
}

__device__ __forceinline__ unsigned mm_tf32(float x) {
  unsigned r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
  return r;
}
__device__ __forceinline__ void mm_split(float x, unsigned& hi, unsigned& lo) {
  hi = mm_tf32(x);
  lo = mm_tf32(x - __uint_as_float(hi));
}
__device__ __forceinline__ void mm_mma(float (&d)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// d = a * b (no accumulator input)
__device__ __forceinline__ void mm_mma_z(float (&d)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
      : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "f"(0.0f));
}
// The three products of one tile and one k-step.  The tensor core aligns its addends by truncation, which
// biases a long accumulation chain at the 1e-6 level; so the main product x_hi*w_hi of every k-step starts from
// zero and is added to the running sum `c` with an ordinary (round-to-nearest) fp32 add, and the two small
// products accumulate in the unit in a sum of their own (`e`, added once at the end), where the same relative
// error is 2^-11 smaller in absolute terms.
__device__ __forceinline__ void mm_mma3(float (&c)[4], float (&e)[4], const unsigned (&ah)[4], const unsigned (&al)[4],
                                        unsigned bh0, unsigned bh1, unsigned bl0, unsigned bl1) {
  float m[4];
  mm_mma_z(m, ah, bh0, bh1);
  mm_mma(e, al, bh0, bh1);
  mm_mma(e, ah, bl0, bl1);
#pragma unroll
  for (int q = 0; q < 4; q++) c[q] += m[q];
}

// Word r of the pack of a layer with weights W[in][out] (row-major) followed by the bias: what k_prep writes.
// Fragment order of mma.m16n8k8: lane = 4 g + t holds b0 = B[k = t][n = g], b1 = B[k = t + 4][n = g].
__device__ __forceinline__ float mm_pack_value(const float* __restrict__ W, int in, int out, int r) {
  const int K = mm_pad8(in), N = mm_pad8(out);
  float v = 0.0f;
  bool lo;
  if (r < 4 * K * N) {
    const bool rev = r >= 2 * K * N;
    if (rev) r -= 2 * K * N;
    const int ntiles = (rev ? K : N) >> 3;
    const int tile = r >> 7, w = r & 127, lane = w >> 2, c = w & 3;
    const int ks = tile / ntiles, n = tile - ks * ntiles, g = lane >> 2, t = lane & 3;
    const int k = ks * 8 + t + ((c & 1) ? 4 : 0), col = n * 8 + g;
    const int i = rev ? col : k, j = rev ? k : col;  // reverse use: B[k = output][n = input] = W[input][output]
    if (i < in && j < out) v = W[(size_t)i * out + j];
    lo = c >= 2;
  } else {
    const int j = r - 4 * K * N;
    return j < out ? W[(size_t)in * out + j] : 0.0f;
  }
  const float hi = __uint_as_float(mm_tf32(v));
  return lo ? __uint_as_float(mm_tf32(v - hi)) : hi;
}

// A fragments of the 16 x 8 block at columns k0.. of a [16][lda] buffer (row = atom), split
__device__ __forceinline__ void mm_load_a(const float* __restrict__ A, int lda, int k0, int g, int t,
                                          unsigned (&ah)[4], unsigned (&al)[4]) {
  const float* p = A + g * lda + k0 + t;
  mm_split(p[0], ah[0], al[0]);
  mm_split(p[8 * lda], ah[1], al[1]);
  mm_split(p[4], ah[2], al[2]);
  mm_split(p[8 * lda + 4], ah[3], al[3]);
}

// C[16][8 ntiles] = A[16][8 ksteps] * B, B from a fragment pack in global memory; TWO: a second left-hand side
// A2 against the same B.  The block's gw warps share the output tiles: this warp owns tiles warp, warp + gw, ...
// and works on NT of them at a time, with the fragments of the next D k-steps already on their way (ring of
// D x NT 16-byte registers per lane).  epi(row, col, c0, c1, d0, d1) receives the values at (row, col) and
// (row, col + 1) of both products.
template <int NT, int D, bool TWO, class Epi>
__device__ __forceinline__ void mm_gemm_w(const float* __restrict__ A1, const float* __restrict__ A2, int lda,
                                          int ksteps, int ntiles, const float4* __restrict__ Bp, int warp, int gw,
                                          int lane, Epi&& epi) {
  const int g = lane >> 2, t = lane & 3;
  for (int nb = warp; nb < ntiles; nb += gw * NT) {
    float c1[NT][4], e1[NT][4], c2[TWO ? NT : 1][4], e2[TWO ? NT : 1][4];
    float4 ring[D][NT];
#pragma unroll
    for (int j = 0; j < NT; j++)
#pragma unroll
      for (int q = 0; q < 4; q++) {
        c1[j][q] = e1[j][q] = 0.0f;
        if (TWO) c2[j][q] = e2[j][q] = 0.0f;
      }
#pragma unroll
    for (int d = 0; d < D; d++)
#pragma unroll
      for (int j = 0; j < NT; j++)
        if (d < ksteps && nb + j * gw < ntiles) ring[d][j] = __ldg(Bp + ((size_t)d * ntiles + nb + j * gw) * 32 + lane);
    for (int ks0 = 0; ks0 < ksteps; ks0 += D) {
#pragma unroll
      for (int d = 0; d < D; d++) {
        const int ks = ks0 + d;
        if (ks < ksteps) {
          unsigned ah[4], al[4], ah2[4], al2[4];
          mm_load_a(A1, lda, ks * 8, g, t, ah, al);
          if (TWO) mm_load_a(A2, lda, ks * 8, g, t, ah2, al2);
#pragma unroll
          for (int j = 0; j < NT; j++) {
            if (nb + j * gw < ntiles) {
              const float4 b = ring[d][j];
              if (ks + D < ksteps)
                ring[d][j] = __ldg(Bp + ((size_t)(ks + D) * ntiles + nb + j * gw) * 32 + lane);
              const unsigned bh0 = __float_as_uint(b.x), bh1 = __float_as_uint(b.y), bl0 = __float_as_uint(b.z),
                             bl1 = __float_as_uint(b.w);
              mm_mma3(c1[j], e1[j], ah, al, bh0, bh1, bl0, bl1);
              if (TWO) mm_mma3(c2[j], e2[j], ah2, al2, bh0, bh1, bl0, bl1);
            }
          }
        }
      }
    }
#pragma unroll
    for (int j = 0; j < NT; j++) {
      if (nb + j * gw < ntiles) {
        const int col = (nb + j * gw) * 8 + 2 * t;
#pragma unroll
        for (int q = 0; q < 4; q++) {
          c1[j][q] += e1[j][q];
          if (TWO) c2[j][q] += e2[j][q];
        }
        epi(g, col, c1[j][0], c1[j][1], TWO ? c2[j][0] : 0.0f, TWO ? c2[j][1] : 0.0f);
        epi(g + 8, col, c1[j][2], c1[j][3], TWO ? c2[j][2] : 0.0f, TWO ? c2[j][3] : 0.0f);
      }
    }
  }
}
// few tiles per warp: a deep ring; many (wide layers): a wider, shallower one
template <bool TWO, class Epi>
__device__ __forceinline__ void mm_gemm(const float* __restrict__ A1, const float* __restrict__ A2, int lda, int ksteps,
                                        int ntiles, const float* __restrict__ Bp, int warp, int gw, int lane,
                                        Epi&& epi) {
  const float4* bp = reinterpret_cast<const float4*>(Bp);
  if (ntiles > 2 * gw) mm_gemm_w<TWO ? 3 : 5, 2, TWO>(A1, A2, lda, ksteps, ntiles, bp, warp, gw, lane, epi);
  else mm_gemm_w<2, 4, TWO>(A1, A2, lda, ksteps, ntiles, bp, warp, gw, lane, epi);
}

// Forward: e_i, the activations for the backward kernel ([block][16][padded widths]) and
// netderiv = d(sum e)/dAF.  Block = 16 atoms, gw = blockDim.x / 32 warps.
__global__ void __launch_bounds__(32 * MM_MAX_WARPS)
    k_mlp_fwd_mma(ModelDev md, int nf, const float* __restrict__ theta, const float* __restrict__ wm, int wm_stride,
                  const float* __restrict__ af, float* __restrict__ acts, float* __restrict__ e_atom,
                  float* __restrict__ netderiv) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __shared__ long long rows[MM_ATOMS];
  const int gw = blockDim.x >> 5;
  int t, q0;
  locate_block(md, nf, MM_ATOMS, t, q0);
  const int nat = nf * md.tipos[t];
  const MmShape S = mm_shape(md, t);
  const int L = S.L, F = S.F, Fm = md.Fmax;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float* X = reinterpret_cast<float*>(smem_raw);
  float* H = X + MM_ATOMS * S.ldx;
  float* C0 = H + MM_ATOMS * S.ldh;
  float* C1 = C0 + MM_ATOMS * S.ldc;
  const float* mu = theta + md.off_mu[t];
  const float* wp = wm + (size_t)t * wm_stride;
  if (threadIdx.x < MM_ATOMS) rows[threadIdx.x] = ml_atom_row(md, t, q0, nat, threadIdx.x);
  __syncthreads();
  chain_wait();  // the pack is older than the preceding kernel; everything read below is its output
  // a warp loads the columns of atoms warp, warp + gw, ...: four atoms' loads in flight together (a store to
  // shared memory between two global loads would order them)
  for (int a0 = warp; a0 < MM_ATOMS; a0 += 4 * gw) {
    for (int i = lane; i < S.ldx; i += 32) {
      float v[4];
#pragma unroll
      for (int q = 0; q < 4; q++) {
        const int a = a0 + q * gw;
        const long long r = a < MM_ATOMS ? rows[a] : -1;
        v[q] = (r >= 0 && i < F) ? af[r * Fm + i] : 1.0f;
      }
      const float m = i < F ? mu[i] : 0.0f;
#pragma unroll
      for (int q = 0; q < 4; q++) {
        const int a = a0 + q * gw;
        if (a < MM_ATOMS) X[a * S.ldx + i] = (rows[a] >= 0 && i < F) ? r_log(v[q] + 1e-3f) - m : 0.0f;
      }
    }
  }
  __syncthreads();
  for (int l = 0; l < L; l++) {
    const float* A = l == 0 ? X : H + S.hoff[l - 1];
    const int lda = l == 0 ? S.ldx : S.ldh;
    const float* lw = wp + S.woff[l];
    const float* bias = lw + 4 * mm_pad8(S.in[l]) * mm_pad8(S.out[l]);
    float* out = H + S.hoff[l];
    const bool act = l < L - 1;
    mm_gemm<false>(A, nullptr, lda, mm_pad8(S.in[l]) >> 3, mm_pad8(S.out[l]) >> 3, lw, warp, gw, lane,
                   [&](int row, int col, float c0, float c1, float, float) {
                     c0 += __ldg(bias + col);
                     c1 += __ldg(bias + col + 1);
                     if (act) { c0 = ml_tanh(c0); c1 = ml_tanh(c1); }
                     *reinterpret_cast<float2*>(out + row * S.ldh + col) = make_float2(c0, c1);
                   });
    __syncthreads();
  }
  {
    const int HsP = S.hoff[L];
    float* ab = acts + (size_t)blockIdx.x * MM_ATOMS * HsP;
    for (int a = warp; a < MM_ATOMS; a += gw)
      for (int c = lane; c < HsP; c += 32) ab[a * HsP + c] = H[a * S.ldh + c];
    if (threadIdx.x < MM_ATOMS && rows[threadIdx.x] >= 0)
      e_atom[rows[threadIdx.x]] = H[threadIdx.x * S.ldh + S.hoff[L - 1]];
  }
  // d(sum e)/dx by the reverse sweep; the factor 1 - h^2 of the layer below is applied as the product leaves the
  // accumulators
  float* cn = C0;
  float* cp = C1;
  for (int idx = threadIdx.x; idx < MM_ATOMS * 8; idx += blockDim.x)
    cn[(idx >> 3) * S.ldc + (idx & 7)] = (idx & 7) == 0 ? 1.0f : 0.0f;
  __syncthreads();
  for (int l = L - 1; l >= 0; l--) {
    const float* lw = wp + S.woff[l] + 2 * mm_pad8(S.in[l]) * mm_pad8(S.out[l]);  // reverse fragments
    const float* hb = l > 0 ? H + S.hoff[l - 1] : nullptr;
    float* dst = cp;
    mm_gemm<false>(cn, nullptr, S.ldc, mm_pad8(S.out[l]) >> 3, mm_pad8(S.in[l]) >> 3, lw, warp, gw, lane,
                   [&](int row, int col, float c0, float c1, float, float) {
                     if (hb) {
                       const float2 h = *reinterpret_cast<const float2*>(hb + row * S.ldh + col);
                       c0 *= 1.0f - h.x * h.x;
                       c1 *= 1.0f - h.y * h.y;
                     }
                     *reinterpret_cast<float2*>(dst + row * S.ldc + col) = make_float2(c0, c1);
                   });
    __syncthreads();
    float* tmp = cn; cn = cp; cp = tmp;
  }
  for (int a0 = warp; a0 < MM_ATOMS; a0 += 4 * gw) {
    for (int i = lane; i < Fm; i += 32) {
      float v[4];
#pragma unroll
      for (int q = 0; q < 4; q++) {
        const int a = a0 + q * gw;
        const long long r = a < MM_ATOMS ? rows[a] : -1;
        v[q] = (r >= 0 && i < F) ? af[r * Fm + i] : 1.0f;
      }
#pragma unroll
      for (int q = 0; q < 4; q++) {
        const int a = a0 + q * gw;
        const long long r = a < MM_ATOMS ? rows[a] : -1;
        if (r >= 0) netderiv[r * Fm + i] = i < F ? cn[a * S.ldc + i] / (v[q] + 1e-3f) : 0.0f;
      }
    }
  }
}

// Backward of  S = sum_a ebar[a] e[a] + sum_{a,c} u[a,c] netderiv[a,c]  with respect to the weights, mu and AF
// (the second term: tangent v = u/(AF + eps) pushed forward, then reversed), and the contraction of dL/dAF with
// the per-atom d(AF)/d(alpha) rows of the fingerprint sweep - as k_mlp_bwd of mlp.cuh.
__global__ void __launch_bounds__(32 * MM_MAX_WARPS)
    k_mlp_bwd_mma(ModelDev md, int nf, const float* __restrict__ theta, const float* __restrict__ wm, int wm_stride,
                  const float* __restrict__ af, const float* __restrict__ acts, const float* __restrict__ ebar,
                  const float* __restrict__ u, const float* __restrict__ vrow, int nv, float* __restrict__ gaf,
                  float* __restrict__ grad) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __shared__ long long rows[MM_ATOMS];
  const int gw = blockDim.x >> 5;
  int t, q0;
  locate_block(md, nf, MM_ATOMS, t, q0);
  const int nat = nf * md.tipos[t];
  const MmShape S = mm_shape(md, t);
  const int L = S.L, F = S.F, Fm = md.Fmax;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, tq = lane & 3;
  float* X = reinterpret_cast<float*>(smem_raw);  // x
  float* V = X + MM_ATOMS * S.ldx;                // tangent on x
  float* GQ = V + MM_ATOMS * S.ldx;               // dS/dx
  float* GP = GQ + MM_ATOMS * S.ldx;              // dS/dv, then dL/dAF
  float* H = GP + MM_ATOMS * S.ldx;               // activations
  float* HD = H + MM_ATOMS * S.ldh;               // tangents of the activations
  float* DQ = HD + MM_ATOMS * S.ldh;  // tangents of the pre-activations, replaced layer by layer by the cotangents on them
  float* DP = DQ + MM_ATOMS * S.ldh;  // cotangents on the tangents of the pre-activations
  const float* mu = theta + md.off_mu[t];
  const float* wp = wm + (size_t)t * wm_stride;
  if (threadIdx.x < MM_ATOMS) rows[threadIdx.x] = ml_atom_row(md, t, q0, nat, threadIdx.x);
  __syncthreads();
  chain_wait();
  {
    const int HsP = S.hoff[L];
    const float* ab = acts + (size_t)blockIdx.x * MM_ATOMS * HsP;
    for (int a0 = warp; a0 < MM_ATOMS; a0 += 4 * gw) {
      for (int i = lane; i < S.ldx; i += 32) {
        float va[4], vu[4];
#pragma unroll
        for (int q = 0; q < 4; q++) {
          const int a = a0 + q * gw;
          const long long r = a < MM_ATOMS ? rows[a] : -1;
          const bool on = r >= 0 && i < F;
          va[q] = on ? af[r * Fm + i] : 1.0f;
          vu[q] = on ? u[r * Fm + i] : 0.0f;
        }
        const float m = i < F ? mu[i] : 0.0f;
#pragma unroll
        for (int q = 0; q < 4; q++) {
          const int a = a0 + q * gw;
          if (a < MM_ATOMS) {
            const bool on = rows[a] >= 0 && i < F;
            const float den = va[q] + 1e-3f;
            X[a * S.ldx + i] = on ? r_log(den) - m : 0.0f;
            V[a * S.ldx + i] = on ? vu[q] / den : 0.0f;
          }
        }
      }
      for (int c = lane; c < S.ldh; c += 32) {
        float vh[4];
#pragma unroll
        for (int q = 0; q < 4; q++) {
          const int a = a0 + q * gw;
          vh[q] = (a < MM_ATOMS && rows[a] >= 0 && c < HsP) ? ab[a * HsP + c] : 0.0f;
        }
#pragma unroll
        for (int q = 0; q < 4; q++) {
          const int a = a0 + q * gw;
          if (a < MM_ATOMS) {
            H[a * S.ldh + c] = vh[q];
            HD[a * S.ldh + c] = 0.0f;
            DQ[a * S.ldh + c] = 0.0f;
            DP[a * S.ldh + c] = 0.0f;
          }
        }
      }
    }
  }
  __syncthreads();
  // forward tangent: AD = HDin W (kept in DQ) ; HD = AD * act'
  for (int l = 0; l < L; l++) {
    const float* A = l == 0 ? V : HD + S.hoff[l - 1];
    const int lda = l == 0 ? S.ldx : S.ldh;
    const int ho = S.hoff[l];
    const bool act = l < L - 1;
    mm_gemm<false>(A, nullptr, lda, mm_pad8(S.in[l]) >> 3, mm_pad8(S.out[l]) >> 3, wp + S.woff[l], warp, gw, lane,
                   [&](int row, int col, float c0, float c1, float, float) {
                     const int o = row * S.ldh + ho + col;
                     *reinterpret_cast<float2*>(DQ + o) = make_float2(c0, c1);
                     if (act) {
                       const float2 h = *reinterpret_cast<const float2*>(H + o);
                       c0 *= 1.0f - h.x * h.x;
                       c1 *= 1.0f - h.y * h.y;
                     }
                     *reinterpret_cast<float2*>(HD + o) = make_float2(c0, c1);
                   });
    __syncthreads();
  }
  // reverse over (h, hd): the cotangents on the output (q = ebar, p = 1) take the place of the last layer's AD
  for (int idx = threadIdx.x; idx < MM_ATOMS * 8; idx += blockDim.x) {
    const int a = idx >> 3, c = idx & 7;
    const long long r = rows[a];
    const int o = a * S.ldh + S.hoff[L - 1] + c;
    DQ[o] = (c == 0 && r >= 0) ? ebar[r / md.N] : 0.0f;
    DP[o] = (c == 0 && r >= 0) ? 1.0f : 0.0f;
  }
  __syncthreads();
  for (int l = L - 1; l >= 0; l--) {
    const float* lw = wp + S.woff[l] + 2 * mm_pad8(S.in[l]) * mm_pad8(S.out[l]);
    const int hb = l > 0 ? S.hoff[l - 1] : 0;
    const bool last = l == 0;
    mm_gemm<true>(DQ + S.hoff[l], DP + S.hoff[l], S.ldh, mm_pad8(S.out[l]) >> 3, mm_pad8(S.in[l]) >> 3, lw, warp, gw,
                  lane, [&](int row, int col, float q0_, float q1_, float p0, float p1) {
                    if (last) {
                      *reinterpret_cast<float2*>(GQ + row * S.ldx + col) = make_float2(q0_, q1_);
                      *reinterpret_cast<float2*>(GP + row * S.ldx + col) = make_float2(p0, p1);
                    } else {
                      // cotangents on (h, hd) of layer l - 1 -> on its pre-activation and that one's tangent
                      const int o = row * S.ldh + hb + col;
                      const float2 h = *reinterpret_cast<const float2*>(H + o);
                      const float2 ad = *reinterpret_cast<const float2*>(DQ + o);
                      const float d0 = 1.0f - h.x * h.x, d1 = 1.0f - h.y * h.y;
                      *reinterpret_cast<float2*>(DQ + o) = make_float2(q0_ * d0 + p0 * (-2.0f * h.x * d0 * ad.x),
                                                                       q1_ * d1 + p1 * (-2.0f * h.y * d1 * ad.y));
                      *reinterpret_cast<float2*>(DP + o) = make_float2(p0 * d0, p1 * d1);
                    }
                  });
    __syncthreads();
  }
  // dL/dAF; kept in GP for the contraction below
  for (int a0 = warp; a0 < MM_ATOMS; a0 += 4 * gw) {
    for (int i = lane; i < Fm; i += 32) {
      float va[4], vu[4];
#pragma unroll
      for (int q = 0; q < 4; q++) {
        const int a = a0 + q * gw;
        const long long r = a < MM_ATOMS ? rows[a] : -1;
        const bool on = r >= 0 && i < F;
        va[q] = on ? af[r * Fm + i] : 1.0f;
        vu[q] = on ? u[r * Fm + i] : 0.0f;
      }
#pragma unroll
      for (int q = 0; q < 4; q++) {
        const int a = a0 + q * gw;
        if (a < MM_ATOMS) {
          const long long r = rows[a];
          float gv = 0.0f;
          if (r >= 0 && i < F) {
            const float den = va[q] + 1e-3f;
            gv = GQ[a * S.ldx + i] / den + GP[a * S.ldx + i] * (-vu[q] / (den * den));
          }
          if (r >= 0) gaf[r * Fm + i] = gv;
          GP[a * S.ldx + i] = gv;
        }
      }
    }
  }
  __syncthreads();
  if (vrow) {
    // dL/dalpha (fingerprint part) = sum_atoms dL/dAF[c(q)] * dAF[c(q)]/dalpha[q] over the block's atoms;
    // alpha2b and alpha3b are contiguous in theta, q runs over both
    const int Fr = md.Fr[t], Fa = md.Fa[t], n2 = md.nt * Fr, nq = n2 + md.C * 3 * Fa;
    for (int q = threadIdx.x; q < nq; q += blockDim.x) {
      const int ch = q < n2 ? (q % Fr) : Fr + ((q - n2) / 3) % Fa;
      int qa;  // position of parameter q in the rows the fingerprint sweep wrote (its accumulator layout)
      if (q < n2) qa = (q / Fr) * md.Frmax + (q % Fr);
      else {
        const int r = q - n2, sc = r / 3, s = sc / Fa;
        qa = md.nt * md.Frmax + (s * md.Famax + (sc - s * Fa)) * 3 + (r - sc * 3);
      }
      float gsum = 0.0f;
#pragma unroll 8
      for (int a = 0; a < MM_ATOMS; a++) {
        const long long r = rows[a];
        if (r >= 0) gsum += GP[a * S.ldx + ch] * vrow[r * nv + qa];
      }
      if (gsum != 0.0f) atomicAdd(grad + md.off_a2[t] + q, gsum);
    }
  }
  // ---- weight gradients of the block's atoms: G_l[i][j] = sum_a hin[a][i] q_l[a][j] + hdin[a][i] p_l[a][j].
  // Units of (layer, 16 features, 2 output tiles) dealt to the warps; A = hin^T read from the [atom][feature]
  // buffers, B = q_l, both split on the fly.
  float* gw_ = grad + md.off_w[t];
  int unit_end[STAFB_MAX_DENSE];
  {
    int tot = 0;
    for (int l = 0; l < STAFB_MAX_DENSE; l++) {
      if (l < L) tot += ((mm_pad8(S.in[l]) + 15) >> 4) * ((mm_pad8(S.out[l]) + 15) >> 4);
      unit_end[l] = tot;
    }
  }
  for (int unit = warp; unit < unit_end[STAFB_MAX_DENSE - 1]; unit += gw) {
    int l = 0;
#pragma unroll
    for (int q = 0; q < STAFB_MAX_DENSE - 1; q++) l += (unit >= unit_end[q]) ? 1 : 0;
    int ubeg = 0;
#pragma unroll
    for (int q = 0; q < STAFB_MAX_DENSE - 1; q++)
      if (q < l) ubeg = unit_end[q];
    const int in = S.in[l], out = S.out[l];
    const int ntiles = mm_pad8(out) >> 3, nch = (ntiles + 1) >> 1;
    const int lu = unit - ubeg, mt = lu / nch, nc = lu - mt * nch;
    const int i0 = mt * 16, j0 = nc * 16;
    const bool two = nc * 2 + 1 < ntiles;  // the second output tile of this unit exists
    const float* Ain = l == 0 ? X : H + S.hoff[l - 1];
    const float* Adi = l == 0 ? V : HD + S.hoff[l - 1];
    const int lda = l == 0 ? S.ldx : S.ldh;
    const float* Bq = DQ + S.hoff[l];
    const float* Bp_ = DP + S.hoff[l];
    float c[2][4], e[2][4];
#pragma unroll
    for (int j = 0; j < 2; j++)
#pragma unroll
      for (int q = 0; q < 4; q++) c[j][q] = e[j][q] = 0.0f;
#pragma unroll
    for (int pr = 0; pr < 2; pr++) {  // the two products: (hin, q) and (hdin, p)
      const float* As = pr ? Adi : Ain;
      const float* Bs = pr ? Bp_ : Bq;
#pragma unroll
      for (int kk = 0; kk < 2; kk++) {  // 8 atoms each
        const float* ap = As + (kk * 8 + tq) * lda + i0 + g;
        unsigned ah[4], al[4];
        mm_split(ap[0], ah[0], al[0]);
        mm_split(ap[8], ah[1], al[1]);
        mm_split(ap[4 * lda], ah[2], al[2]);
        mm_split(ap[4 * lda + 8], ah[3], al[3]);
        const float* bp = Bs + (kk * 8 + tq) * S.ldh + j0 + g;
#pragma unroll
        for (int j = 0; j < 2; j++) {
          if (j == 0 || two) {
            unsigned bh0, bl0, bh1, bl1;
            mm_split(bp[j * 8], bh0, bl0);
            mm_split(bp[4 * S.ldh + j * 8], bh1, bl1);
            mm_mma3(c[j], e[j], ah, al, bh0, bh1, bl0, bl1);
          }
        }
      }
    }
    const int woff = md.w_off(t, l);
#pragma unroll
    for (int j = 0; j < 2; j++) {
      if (j == 0 || two) {
        const int col = j0 + j * 8 + 2 * tq;
#pragma unroll
        for (int q = 0; q < 4; q++) {
          const int i = i0 + g + ((q & 2) ? 8 : 0), jj = col + (q & 1);
          if (i < in && jj < out) atomicAdd(gw_ + woff + i * out + jj, c[j][q] + e[j][q]);
        }
      }
    }
  }
  // bias gradients and d/dmu: column sums over the block's atoms
  for (int l = 0; l < L; l++) {
    const int in = S.in[l], out = S.out[l];
    const float* q = DQ + S.hoff[l];
    const int woff = md.w_off(t, l);
    for (int j = threadIdx.x; j < out; j += blockDim.x) {
      float gs = 0.0f;
#pragma unroll
      for (int a = 0; a < MM_ATOMS; a++) gs += q[a * S.ldh + j];
      atomicAdd(gw_ + woff + in * out + j, gs);
    }
  }
  for (int i = threadIdx.x; i < F; i += blockDim.x) {
    float gs = 0.0f;
#pragma unroll
    for (int a = 0; a < MM_ATOMS; a++) gs -= GQ[a * S.ldx + i];
    atomicAdd(grad + md.off_mu[t] + i, gs);
  }
}
