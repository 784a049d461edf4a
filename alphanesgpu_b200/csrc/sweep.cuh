// Sweep kernels of the fused path (included by fused.cu inside namespace stafb): atomic fingerprints, forces and
// the backward of the forces, each as one pass over the triplets of every central atom.
//
// One warp owns one central atom.  Its neighbour record (common.cuh: unit vectors, cutoffs, radial descriptors,
// neighbour ids, grouped by species) and the per-species parameter block that k_prep packs once per evaluation
// arrive in shared memory by two bulk asynchronous copies that complete on an mbarrier; nothing about the
// geometry is recomputed here except the angle of a pair.
//
// Triplets are enumerated per species-pair class (ta <= tb) rather than in the reference's j<k slot order: inside
// a class every triplet uses the same parameter row (row = type_j + type_k,
// STAF/src/fingerprint/ang/reforce.cu.cc:56), so the channel loop is uniform across the warp and channels whose
// squared embedding is zero are skipped for the whole class.  exp(a1*sj + a2*sk) is formed as a product of
// per-neighbour factors exp(a1*sj), exp(a2*sk) tabulated once per (class, channel chunk); in fp32 all
// exponentials are base-2 (one MUFU.EX2) with parameters pre-scaled by log2(e), two channels per packed
// instruction.  The force sweep walks ORDERED pairs so that every lane accumulates the force on "its" neighbour
// in registers; the other sweeps walk unordered pairs and reduce per-lane sums with a transposing butterfly.
//
// Math: STAF/src/fingerprint, force, grad_finger, grad_force (rad and ang) reforce.cu.cc and
// STAF/staf_models/staf_model.py:168-258 of the reference (see include/stafb.h).
#pragma once

constexpr int MAXP = 4;  // channel PAIRS processed per pass over the pairs of a class
// Exponential tables: entry (neighbour k, channel pair lp) at tab4[k * TSTR + lp].  Neighbour-major, so that the
// entries of one neighbour are at constant offsets from one address; the odd stride (5 x 16 bytes) keeps the
// 16-byte loads of lanes on consecutive neighbours free of bank conflicts.
constexpr int TSTR = MAXP + 1;

// ---- bulk asynchronous copy global -> shared, completion on an mbarrier (this GPU's own memory only)
__device__ __forceinline__ unsigned smem_addr(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(unsigned bar, unsigned arrivals) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(arrivals) : "memory");
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(unsigned bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// dst, src 16-byte aligned; bytes a multiple of 16
__device__ __forceinline__ void bulk_g2s(unsigned dst, const void* src, unsigned bytes, unsigned bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
               "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}
// Bounded wait for a phase of the barrier; false if the copies did not land (the caller records a status and
// leaves, it never spins for ever).
__device__ __forceinline__ bool mbar_wait(unsigned bar, unsigned parity) {
  for (int it = 0; it < (1 << 24); it++) {
    unsigned ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    if (ok) return true;
  }
  return false;
}

// 2^x for a pre-scaled argument: one MUFU.EX2 (results below 2^-126 flush to zero; arguments here are products
// of exponents of magnitude <= ~10 with cutoff values in [0,1], far from overflow)
__device__ __forceinline__ float ex2_fast(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
template <class T> struct Ex;
template <> struct Ex<float> {
  static __host__ __device__ __forceinline__ float scale() { return 1.4426950408889634f; }
  static __device__ __forceinline__ float f(float x) { return ex2_fast(x); }
};
template <> struct Ex<double> {
  static __host__ __device__ __forceinline__ double scale() { return 1.0; }
  static __device__ __forceinline__ double f(double x) { return exp(x); }
};

// Two-channel packed arithmetic.  On sm_100 a float2 multiply / add / fma is ONE instruction (__fmul2_rn,
// __fadd2_rn, __ffma2_rn), so the channel loops carry two channels per instruction; double pairs are two scalar
// operations.
__device__ __forceinline__ float2 p_mul(float2 a, float2 b) { return __fmul2_rn(a, b); }
__device__ __forceinline__ float2 p_add(float2 a, float2 b) { return __fadd2_rn(a, b); }
__device__ __forceinline__ float2 p_fma(float2 a, float2 b, float2 c) { return __ffma2_rn(a, b, c); }
__device__ __forceinline__ double2 p_mul(double2 a, double2 b) { return make_double2(a.x * b.x, a.y * b.y); }
__device__ __forceinline__ double2 p_add(double2 a, double2 b) { return make_double2(a.x + b.x, a.y + b.y); }
__device__ __forceinline__ double2 p_fma(double2 a, double2 b, double2 c) {
  return make_double2(a.x * b.x + c.x, a.y * b.y + c.y);
}
__device__ __forceinline__ float2 mk2(float x, float y) { return make_float2(x, y); }
__device__ __forceinline__ double2 mk2(double x, double y) { return make_double2(x, y); }
__device__ __forceinline__ float2 p_ex(float2 a) { return make_float2(Ex<float>::f(a.x), Ex<float>::f(a.y)); }
__device__ __forceinline__ double2 p_ex(double2 a) { return make_double2(Ex<double>::f(a.x), Ex<double>::f(a.y)); }

// AFV = fingerprints that also leave d(AF)/d(alpha) per atom (training)
enum { MODE_AF = 0, MODE_FORCE = 1, MODE_FGRAD = 2, MODE_AFV = 4 };

// Resident one-warp blocks per SM the kernels are compiled for (caps the registers per thread at
// 65536 / (32 * blocks)); the hardware holds at most 32 blocks per SM.
// fp32: 96 registers, five warps per scheduler = 20 blocks per SM (the shared memory of a block allows the same).  A
// batch of 4 x 768 atoms is 20.8 blocks per SM; the few that do not fit start as the first ones retire.  Capping at
// 80 registers for 24 blocks was measured: spills, and no gain in the chained step.
template <int MODE, size_t ES> struct SweepMinBlocks { static constexpr int value = 20; };
template <> struct SweepMinBlocks<MODE_AF, 8> { static constexpr int value = 16; };          // <= 128
template <> struct SweepMinBlocks<MODE_AFV, 8> { static constexpr int value = 12; };         // <= 168
template <> struct SweepMinBlocks<MODE_FORCE, 8> { static constexpr int value = 8; };        // no spills at <= 255
template <> struct SweepMinBlocks<MODE_FGRAD, 8> { static constexpr int value = 8; };        // <= 255

// ---- per-species parameter block (global memory, written by k_prep at the start of every evaluation; a sweep
// copies the block of its central species into shared memory).  Byte offsets inside a block:
//   [0, 32)  int nact[8]            active channels (squared embedding != 0) of class s = ta + tb
//   actc     uchar [ncls][Famax]    their channel numbers, compacted
//   chq      T4 [ncls][maxp]        channel pair (2p, 2p+1) of the compacted list: alpha1 x2, alpha2 x2
//   chr      T4 [ncls][maxp]        beta x2, beta*log2(e) x2
//   che      T2 [ncls][maxp]        squared embedding x2 (an odd count is padded with an all-zero channel)
//   rpar     T4 [nt][Frmax]         radial channels: alpha2b*log2(e), alpha2b, squared embedding, 0
struct SparLayout {
  int actc, chq, chr, che, rpar, total, maxp;
};
template <class T>
static inline SparLayout spar_layout(const ModelDev& d) {
  SparLayout L;
  int o = 32;
  auto take = [&](int bytes) { int r = o; o += (bytes + 15) & ~15; return r; };
  L.maxp = (d.Famax + 1) / 2 > 0 ? (d.Famax + 1) / 2 : 1;
  L.actc = take(d.ncls * (d.Famax > 0 ? d.Famax : 1));
  L.chq = take(d.ncls * L.maxp * 4 * (int)sizeof(T));
  L.chr = take(d.ncls * L.maxp * 4 * (int)sizeof(T));
  L.che = take(d.ncls * L.maxp * 2 * (int)sizeof(T));
  L.rpar = take(d.nt * (d.Frmax > 0 ? d.Frmax : 1) * 4 * (int)sizeof(T));
  L.total = o;
  return L;
}

// Fills the block of (species t, class s): one warp; lanes over channels, ballot compaction of the active ones.
template <class T>
__device__ __forceinline__ void spar_fill_class(const ModelDev& md, const SparLayout& sl, unsigned char* blk, int t,
                                                int s, const T* __restrict__ theta, const T* __restrict__ emb,
                                                int lane) {
  typedef typename Vec4<T>::type T4;
  typedef typename Vec2<T>::type T2;
  const int Fa = md.Fa[t], Fr = md.Fr[t], nt = md.nt;
  const T* a3 = theta + md.off_a3[t] + (size_t)s * 3 * Fa;
  const T* e3 = emb + md.off_emb[t] + nt * Fr + (size_t)s * Fa;
  unsigned char* actc = blk + sl.actc + s * md.Famax;
  T* chq = reinterpret_cast<T*>(blk + sl.chq) + (size_t)s * sl.maxp * 4;
  T* chr = reinterpret_cast<T*>(blk + sl.chr) + (size_t)s * sl.maxp * 4;
  T* che = reinterpret_cast<T*>(blk + sl.che) + (size_t)s * sl.maxp * 2;
  const unsigned lt = (1u << lane) - 1u;
  const T SC = Ex<T>::scale();
  int nact = 0;
  for (int c0 = 0; c0 < Fa; c0 += 32) {
    const int c = c0 + lane;
    const T ee = c < Fa ? e3[c] : T(0);
    const bool p = ee != T(0);
    const unsigned bal = __ballot_sync(0xffffffffu, p);
    if (p) {
      const int slot = nact + __popc(bal & lt), pr = slot >> 1, h = slot & 1;
      const T al1 = a3[3 * c], al2 = a3[3 * c + 1], be = a3[3 * c + 2];
      actc[slot] = (unsigned char)c;
      chq[pr * 4 + h] = al1; chq[pr * 4 + 2 + h] = al2;
      chr[pr * 4 + h] = be;  chr[pr * 4 + 2 + h] = be * SC;
      che[pr * 2 + h] = ee;
    }
    nact += __popc(bal);
  }
  if (lane == 0) {
    reinterpret_cast<int*>(blk)[s] = nact;
    if (nact & 1) {  // the partner of the last channel: a channel that contributes nothing
      const int pr = nact >> 1;
      chq[pr * 4 + 1] = T(0); chq[pr * 4 + 3] = T(0);
      chr[pr * 4 + 1] = T(0); chr[pr * 4 + 3] = T(0);
      che[pr * 2 + 1] = T(0);
    }
  }
}

template <class T>
__device__ __forceinline__ void spar_fill_radial(const ModelDev& md, const SparLayout& sl, unsigned char* blk, int t,
                                                 const T* __restrict__ theta, const T* __restrict__ emb, int idx) {
  const int Fr = md.Fr[t], q = idx / Fr, c = idx - q * Fr;
  T* rp = reinterpret_cast<T*>(blk + sl.rpar) + ((size_t)q * md.Frmax + c) * 4;
  const T al = theta[md.off_a2[t] + idx];
  rp[0] = al * Ex<T>::scale(); rp[1] = al; rp[2] = emb[md.off_emb[t] + idx]; rp[3] = T(0);
}

// The virial of a frame is accumulated by every centre of the frame: 9 words would take one atomic add per atom
// each (24,576 on one address for a large box), so every component has VIR_SLOTS words, a centre adds to slot
// (its index mod VIR_SLOTS) and the readers sum the slots.  Layout [frame][9][VIR_SLOTS] doubles.
constexpr int VIR_SLOTS = 32;
__device__ __forceinline__ double vir_total(const double* __restrict__ vacc, int frame, int q) {
  const double* p = vacc + ((size_t)frame * 9 + q) * VIR_SLOTS;
  double w = 0.0;
#pragma unroll 8
  for (int s = 0; s < VIR_SLOTS; s++) w += p[s];
  return w;
}

template <class T>
struct SweepArgs {
  const unsigned char* rows;  // [nf, N] neighbour records
  int row_stride;             // bytes
  int nr, nf, nall;           // nall: atoms per frame in the force / cotangent arrays (>= N: ghosts)
  const unsigned char* spar;  // [nt] parameter blocks
  int spar_stride;
  SparLayout sl;
  const T* chan_in;  // FORCE/FGRAD: netderiv[nf,N,Fmax]
  const T* force;    // FGRAD: forces [nf,3*nall] and their labels; dL/dF = fscale * L'(force - label) with L the
  const T* flab;     //        Huber (loss_kind 0) or the squared error
  T fscale;
  int loss_kind;
  T* out;            // AF/AFV: af[nf,N,Fmax]; FORCE: force[nf,3*nall]; FGRAD: gradnet[nf,N,Fmax]
  T* grad;           // FGRAD: flat parameter gradient (accumulated)
  T* vout;           // AFV: d(AF)/d(alpha) rows [nf,N,nv] in the accumulator layout (alpha2b[nt,Frmax] | alpha3b[C,3*Famax])
  int nv;
  double* vir;       // FORCE with VIR: virial accumulators [nf,9,VIR_SLOTS]
  const double* vacc;  // FGRAD with a virial loss: the accumulators the force sweep filled, the labels [nf,9] and
  const T* vlab;       //        the loss's scale: dL/dW = vscale * L'(W - label)
  T vscale;
  int* status;
};

// shared-memory layout of a sweep block (byte offsets)
struct SweepSmem {
  int row, spar, tab, xtra, acc, rsum, wch, red, mbar, total;
};
template <class T>
static inline SweepSmem sweep_smem(const ModelDev& d, const SparLayout& sl, int nr, int mode) {
  SweepSmem L;
  int o = 0;
  auto take = [&](int bytes) { int r = o; o += (bytes + 15) & ~15; return r; };
  const int es = (int)sizeof(T);
  L.row = take(row_stride_bytes(nr, es));
  L.spar = take(sl.total);
  L.tab = take(TSTR * nr * 4 * es);
  L.xtra = take(mode == MODE_FORCE ? 3 * nr * es : (mode == MODE_FGRAD ? 4 * nr * es : 0));
  L.acc = take((d.nt * d.Frmax + d.C * 3 * d.Famax + d.Famax) * es);
  L.rsum = take(d.nt * (d.Frmax > 0 ? d.Frmax : 1) * es);
  L.wch = take(mode == MODE_FORCE ? d.ncls * sl.maxp * 2 * es : 0);
  L.red = take(32 * es);  // group offsets
  L.mbar = take(16);
  L.total = o;
  return L;
}

// Sums NV per-lane values over the 32 lanes of a warp.  Every step halves the number of values a lane
// still carries (lanes with the step's bit set keep the upper half and hand over the lower one), so
// NV-1 shuffles replace 5*NV; once one value is left the remaining steps are a plain butterfly.
// On return lane L holds the total of value index L >> log2(32 / NV).  NV is a power of two <= 32.
template <class T, int NV>
__device__ __forceinline__ T multi_reduce(T (&v)[NV], int lane) {
  static_assert(NV == 1 || NV == 2 || NV == 4 || NV == 8 || NV == 16 || NV == 32, "NV must be a power of two");
  int off = 16;
#pragma unroll
  for (int half = NV / 2; half >= 1; half >>= 1) {
    const bool up = (lane & off) != 0;
#pragma unroll
    for (int i = 0; i < half; i++) {
      const T keep = up ? v[i + half] : v[i];
      const T send = up ? v[i] : v[i + half];
      v[i] = keep + __shfl_xor_sync(0xffffffffu, send, off);
    }
    off >>= 1;
  }
  T r = v[0];
  for (; off >= 1; off >>= 1) r += __shfl_xor_sync(0xffffffffu, r, off);
  return r;
}

// Pairs of a class as a rectangle of rows x cols walked 32 positions at a time without divisions.  Two different
// species (SAME == false): rows = neighbours of ta, cols = neighbours of tb.  One species with n neighbours: the
// strict upper triangle j < k folded into a rectangle - row r of the triangle (n-1-r entries) is followed by row
// n-1-r (n even) or n-2-r (n odd), which together have n-1 (n) entries.
template <bool SAME>
struct PairWalk {
  int r, c, cols, q32, r32, nm1, odd;
  __device__ __forceinline__ void init(int na, int nb, int lane) {
    odd = na & 1;
    nm1 = na - 1;
    cols = SAME ? (odd ? na : na - 1) : nb;
    if (cols < 1) cols = 1;
    r = lane / cols;
    c = lane - r * cols;
    q32 = 32 / cols;
    r32 = 32 - q32 * cols;
  }
  __device__ __forceinline__ static int count(int na, int nb) { return SAME ? na * (na - 1) / 2 : na * nb; }
  __device__ __forceinline__ void get(int& j, int& k) const {
    if (SAME) {
      const bool first = c < nm1 - r;
      j = first ? r : nm1 - odd - r;
      k = first ? r + 1 + c : c + 1 - odd;
    } else {
      j = r;
      k = c;
    }
  }
  __device__ __forceinline__ void step() {
    r += q32;
    c += r32;
    if (c >= cols) { c -= cols; r++; }
  }
};

// ---- unordered pairs: fingerprints (AF), fingerprints + d(AF)/d(alpha) (AFV), backward of the forces (FGRAD).
// Per-lane sums r[v][lp] (v = 0: fingerprint / gradnet, 1..3: alpha1, alpha2, beta terms) for NCHP channel pairs.
template <class T, int MODE, int NCHP, bool SAME>
__device__ __forceinline__ void pairs_unordered(const typename Vec4<T>::type* __restrict__ U,
                                                const typename Vec4<T>::type* __restrict__ V,
                                                const typename Vec4<T>::type* __restrict__ dF,
                                                const typename Vec4<T>::type* __restrict__ tab4, int nr,
                                                const typename Vec4<T>::type* __restrict__ chq,
                                                const typename Vec4<T>::type* __restrict__ chr, int oa, int ob,
                                                int na_, int nb_, int lane,
                                                typename Vec2<T>::type (&r0)[NCHP], typename Vec2<T>::type (&r1)[NCHP],
                                                typename Vec2<T>::type (&r2)[NCHP],
                                                typename Vec2<T>::type (&r3)[NCHP]) {
  typedef typename Vec4<T>::type T4;
  typedef typename Vec2<T>::type T2;
#pragma unroll
  for (int lp = 0; lp < NCHP; lp++) r0[lp] = r1[lp] = r2[lp] = r3[lp] = mk2(T(0), T(0));
  const T2 one2 = mk2(T(1), T(1));
  const int np = PairWalk<SAME>::count(na_, nb_);
  PairWalk<SAME> pw;
  pw.init(na_, nb_, lane);
  // beta*log2(e) of every channel pair stays in registers in the fingerprint modes
  T2 bsc[NCHP];
  if (MODE != MODE_FGRAD) {
#pragma unroll
    for (int lp = 0; lp < NCHP; lp++) { const T4 cr = chr[lp]; bsc[lp] = mk2(cr.z, cr.w); }
  }
  // pairs in flight per lane: two hide the shared-memory and exponential latencies of the fingerprint loops; the
  // force-backward loop is too large for that (its unrolled body falls out of the instruction cache)
  constexpr int PAIR_UNROLL = (MODE == MODE_FGRAD) ? 1 : 2;
#pragma unroll PAIR_UNROLL
  for (int p = lane; p < np; p += 32) {
    int jj, kk;
    pw.get(jj, kk);
    pw.step();
    const int j = oa + jj, k = ob + kk;
    const T4 uj = U[j], uk = U[k];
    const T fcj = uj.w, fck = uk.w;
    const T cs = uj.x * uk.x + uj.y * uk.y + uj.z * uk.z;
    const T half = T(0.5) * cs + T(0.5);
    const T tt = half * fcj * fck;
    const T2 tt2 = mk2(tt, tt), fcj2 = mk2(fcj, fcj), fck2 = mk2(fck, fck);
    if (MODE != MODE_FGRAD) {
#pragma unroll
      for (int lp = 0; lp < NCHP; lp++) {
        const T4 A = tab4[j * TSTR + lp], B = tab4[k * TSTR + lp];
        const T2 S1 = p_mul(mk2(A.z, A.w), mk2(B.x, B.y));  // exp(a2*sj + a1*sk)
        const T2 S2 = p_mul(mk2(A.x, A.y), mk2(B.z, B.w));  // exp(a1*sj + a2*sk)
        const T2 cm = p_mul(p_ex(p_mul(bsc[lp], tt2)), tt2);  // t*exp(beta*t)
        const T2 ss = p_add(S1, S2);
        r0[lp] = p_fma(cm, ss, r0[lp]);  // the channel coefficient is applied after the reduction
        if (MODE == MODE_AFV) {
          r1[lp] = p_fma(cm, p_fma(S2, fcj2, p_mul(S1, fck2)), r1[lp]);
          r2[lp] = p_fma(cm, p_fma(S2, fck2, p_mul(S1, fcj2)), r2[lp]);
          r3[lp] = p_fma(p_mul(cm, tt2), ss, r3[lp]);
        }
      }
    } else {
      // Backward of the triplet force for the cotangent dF_k = Fbar_k - Fbar_i (dF.w = dF . u).  With
      //   Q  = d(t)/d(positions) . dF  (symmetric in j,k),  Pj = fc'_j (dF_j . u_j),  Pk likewise,
      //   Z1 = E exp(a1 sj + a2 sk), Z2 = E exp(a2 sj + a1 sk), E = exp(beta t), g = 1 + beta t,
      //   H1 = g Q/2 + (t/2)(a1 Pj + a2 Pk),  H2 = g Q/2 + (t/2)(a1 Pk + a2 Pj)
      // the channel's gradnet term is  Z1 H1 + Z2 H2  (the two orderings of the pair) and the parameter terms are
      // its derivatives:  d/da1 = Z1 (sj H1 + t Pj/2) + Z2 (sk H2 + t Pk/2),  d/da2 with sj, sk and Pj, Pk
      // exchanged inside each bracket,  d/dbeta = t [Z1 (H1 + Q/2) + Z2 (H2 + Q/2)]
      // (STAF/src/grad_force/ang/reforce.cu.cc:47-231).
      const T4 pj = V[j], pk = V[k];
      const T hf = T(0.5) * fcj * fck;
      const T ajk = hf * pj.x, akj = hf * pk.x;
      const T bjk = -cs * ajk + half * pj.y * fck;
      const T bkj = -cs * akj + half * pk.y * fcj;
      const T4 dFj = dF[j], dFk = dF[k];
      const T djuk = dFj.x * uk.x + dFj.y * uk.y + dFj.z * uk.z;
      const T dkuj = dFk.x * uj.x + dFk.y * uj.y + dFk.z * uj.z;
      const T Qh = T(0.5) * (ajk * djuk + bjk * dFj.w + akj * dkuj + bkj * dFk.w);
      const T Pjh = T(0.5) * tt * pj.y * dFj.w;
      const T Pkh = T(0.5) * tt * pk.y * dFk.w;
      const T2 Qh2 = mk2(Qh, Qh), Pj2 = mk2(Pjh, Pjh), Pk2 = mk2(Pkh, Pkh);
#pragma unroll
      for (int lp = 0; lp < NCHP; lp++) {
        const T4 A = tab4[j * TSTR + lp], B = tab4[k * TSTR + lp], cq = chq[lp], cr = chr[lp];
        const T2 al1 = mk2(cq.x, cq.y), al2 = mk2(cq.z, cq.w);
        const T2 E = p_ex(p_mul(mk2(cr.z, cr.w), tt2));
        const T2 Z1 = p_mul(E, p_mul(mk2(A.x, A.y), mk2(B.z, B.w)));
        const T2 Z2 = p_mul(E, p_mul(mk2(A.z, A.w), mk2(B.x, B.y)));
        const T2 gQ = p_mul(p_fma(mk2(cr.x, cr.y), tt2, one2), Qh2);
        const T2 H1 = p_fma(al1, Pj2, p_fma(al2, Pk2, gQ)), H2 = p_fma(al1, Pk2, p_fma(al2, Pj2, gQ));
        r0[lp] = p_fma(Z1, H1, p_fma(Z2, H2, r0[lp]));
        r1[lp] = p_fma(Z1, p_fma(fcj2, H1, Pj2), p_fma(Z2, p_fma(fck2, H2, Pk2), r1[lp]));
        r2[lp] = p_fma(Z1, p_fma(fck2, H1, Pk2), p_fma(Z2, p_fma(fcj2, H2, Pj2), r2[lp]));
        r3[lp] = p_fma(tt2, p_fma(Z1, p_add(H1, Qh2), p_mul(Z2, p_add(H2, Qh2))), r3[lp]);
      }
    }
  }
}

// ---- ordered pairs (owner j, partner k): forces.  The list of an owner's partners is cut into S segments and
// every lane takes one (owner, segment): the owner's data - including its table entries already multiplied by the
// channel weights - and its force accumulator stay in registers for the whole segment, all lanes run the same
// number of iterations, and the accumulators are flushed once per round (S lanes share an owner).  S in 1..4 is
// chosen per class to fill the 32 lanes.  fo[k*3 + a]: force on neighbour k; (fix, fiy, fiz): on the centre.
template <class T, int NCHP, bool SAME>
__device__ __forceinline__ void pairs_force(const typename Vec4<T>::type* __restrict__ U,
                                            const typename Vec4<T>::type* __restrict__ V,
                                            const typename Vec4<T>::type* __restrict__ tab4,
                                            const typename Vec4<T>::type* __restrict__ chq,
                                            const typename Vec4<T>::type* __restrict__ chr,
                                            const typename Vec2<T>::type* __restrict__ wch, int oo, int op, int no,
                                            int npt, int lane, T* __restrict__ fo, T& fix, T& fiy, T& fiz) {
  typedef typename Vec4<T>::type T4;
  typedef typename Vec2<T>::type T2;
  if (no <= 0 || npt <= 0) return;
  // segments per owner: fewest (iterations + 2) * rounds; the 2 stands for loading the owner and flushing
  int S = 1, seg = npt, best = 0x7fffffff;
#pragma unroll
  for (int s = 1; s <= 4; s++) {
    const int sg = (npt + s - 1) / s, rounds = (no * s + 31) >> 5, cost = rounds * (sg + 2);
    if (cost < best) { best = cost; S = s; seg = sg; }
  }
  constexpr int FORCE_UNROLL = sizeof(T) == 4 ? 2 : 1;  // two partners in flight where the registers allow it
  const int nseg = no * S;
  const T2 one2 = mk2(T(1), T(1));
  for (int base = 0; base < nseg; base += 32) {
    const int sidx = base + lane;
    const bool active = sidx < nseg;
    const int ow = active ? ((S == 1) ? sidx : (S == 2) ? (sidx >> 1) : (S == 4) ? (sidx >> 2) : (sidx * 21846) >> 16) : 0;
    const int k0 = (sidx - ow * S) * seg;
    const int j = oo + ow;
    const T4 uj = U[j];
    const T4 vj = V[j];
    const T rinvj = vj.x, gfcj = vj.y;
    T2 a1w[NCHP], a2w[NCHP], b1w[NCHP], b2w[NCHP];  // w*A1_j, w*A2_j, alpha1*w*A1_j, alpha2*w*A2_j
#pragma unroll
    for (int lp = 0; lp < NCHP; lp++) {
      const T4 A = tab4[j * TSTR + lp], cq = chq[lp];
      const T2 w = wch[lp];
      a1w[lp] = p_mul(mk2(A.x, A.y), w);
      a2w[lp] = p_mul(mk2(A.z, A.w), w);
      b1w[lp] = p_mul(mk2(cq.x, cq.y), a1w[lp]);
      b2w[lp] = p_mul(mk2(cq.z, cq.w), a2w[lp]);
    }
    T ax = T(0), ay = T(0), az = T(0), as = T(0);
    // this lane's partners [k0, k1); for one species the owner itself is skipped: partner kb >= ow is row kb + 1
    const int k1 = active ? ((k0 + seg < npt) ? k0 + seg : npt) : k0;
#pragma unroll FORCE_UNROLL
    for (int kb = k0; kb < k1; kb++) {
      {
        const int k = op + kb + ((SAME && kb >= ow) ? 1 : 0);
        const T4 uk = U[k];
        const T cs = uj.x * uk.x + uj.y * uk.y + uj.z * uk.z;
        const T half = T(0.5) * cs + T(0.5);
        const T tt = half * uj.w * uk.w;
        const T2 tt2 = mk2(tt, tt);
        T2 D2 = mk2(T(0), T(0)), BJ2 = mk2(T(0), T(0));
#pragma unroll
        for (int lp = 0; lp < NCHP; lp++) {
          const T4 B = tab4[k * TSTR + lp], cr = chr[lp];
          const T2 A1k = mk2(B.x, B.y), A2k = mk2(B.z, B.w);
          const T2 Ex2 = p_ex(p_mul(mk2(cr.z, cr.w), tt2));
          const T2 sum = p_fma(a1w[lp], A2k, p_mul(a2w[lp], A1k));            // w (S2 + S1)
          D2 = p_fma(p_mul(p_fma(mk2(cr.x, cr.y), tt2, one2), Ex2), sum, D2);  // w e^{bt} (1 + bt) (S1 + S2)
          BJ2 = p_fma(Ex2, p_fma(b1w[lp], A2k, p_mul(b2w[lp], A1k)), BJ2);     // w e^{bt} (a1 S2 + a2 S1)
        }
        const T D = D2.x + D2.y, BJ = (BJ2.x + BJ2.y) * tt;
        // f_ij = cjk*u_k + (...)*u_j
        const T cjk = D * T(0.5) * uj.w * uk.w * rinvj;
        ax += cjk * uk.x; ay += cjk * uk.y; az += cjk * uk.z;
        as += -cs * cjk + gfcj * (D * half * uk.w + BJ);
      }
    }
    if (active) {
      const T fx = ax + as * uj.x, fy = ay + as * uj.y, fz = az + as * uj.z;
      atomicAdd(&fo[j * 3 + 0], fx);
      atomicAdd(&fo[j * 3 + 1], fy);
      atomicAdd(&fo[j * 3 + 2], fz);
      fix -= fx; fiy -= fy; fiz -= fz;
    }
  }
}

// One block of one warp per central atom.  VIR (force mode only) adds the virial; it is a template parameter so
// that the training step's force sweep does not carry its registers.
template <class T, int MODE, bool VIR>
__global__ void __launch_bounds__(32, SweepMinBlocks<MODE, sizeof(T)>::value)
    k_sweep(ModelDev md, SweepArgs<T> a, SweepSmem L) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  typedef typename Vec4<T>::type T4;
  typedef typename Vec2<T>::type T2;
  constexpr bool IS_AF = (MODE == MODE_AF || MODE == MODE_AFV);
  constexpr int ES = (int)sizeof(T);
  const int lane = threadIdx.x;
  int t, b, i;
  if (!locate_atom(md, a.nf, 1, 0, t, b, i)) return;
  const int N = md.N, nr = a.nr, nt = md.nt;
  const int Fr = md.Fr[t], Fa = md.Fa[t], Fmax = md.Fmax, Frmax = md.Frmax, Famax = md.Famax;
  const size_t gi = (size_t)b * N + i;
  const SparLayout& sl = a.sl;
  unsigned char* rowp = smem_raw + L.row;
  const T4* U = reinterpret_cast<const T4*>(rowp);
  const T4* V = reinterpret_cast<const T4*>(rowp + row_off_v(nr, ES));
  const int* ids = reinterpret_cast<const int*>(rowp + row_off_id(nr, ES));
  const int* hdr = reinterpret_cast<const int*>(rowp + row_off_hdr(nr, ES));
  unsigned char* spb = smem_raw + L.spar;
  const int* nact_s = reinterpret_cast<const int*>(spb);
  const unsigned char* actc = spb + sl.actc;
  const T4* chq_all = reinterpret_cast<const T4*>(spb + sl.chq);
  const T4* chr_all = reinterpret_cast<const T4*>(spb + sl.chr);
  const T2* che_all = reinterpret_cast<const T2*>(spb + sl.che);
  const T4* rpar = reinterpret_cast<const T4*>(spb + sl.rpar);
  T4* tab4 = reinterpret_cast<T4*>(smem_raw + L.tab);
  T* xtra = reinterpret_cast<T*>(smem_raw + L.xtra);
  T* acc = reinterpret_cast<T*>(smem_raw + L.acc);
  T* rsum = reinterpret_cast<T*>(smem_raw + L.rsum);
  T2* wch_all = reinterpret_cast<T2*>(smem_raw + L.wch);
  int* off = reinterpret_cast<int*>(smem_raw + L.red);  // [STAFB_MAX_TYPES + 1]
  const unsigned bar = smem_addr(smem_raw + L.mbar);
  // accumulator regions: the first nv entries are the d(AF)/d(alpha) row of the AFV mode
  const int ACC_A2 = 0;                      // [nt*Frmax]  alpha2b terms
  const int ACC_A3 = nt * Frmax;             // [C*3*Famax] alpha3b terms
  const int ACC_GN = ACC_A3 + md.C * 3 * Famax;  // [Famax]  fingerprints (AF, AFV) / gradnet (FGRAD)
  const int NACC = ACC_GN + Famax;

  // The neighbour record is at least two kernels old (it belongs to the neighbour kernel of this batch), and so is
  // the parameter block except in the fingerprint sweep, which directly follows k_prep.
  if (lane == 0) mbar_init(bar, 2);
  __syncwarp();
  if (lane == 0) {
    mbar_expect_tx(bar, (unsigned)a.row_stride);
    bulk_g2s(smem_addr(rowp), a.rows + gi * (size_t)a.row_stride, (unsigned)a.row_stride, bar);
    if (!IS_AF) {
      mbar_expect_tx(bar, (unsigned)sl.total);
      bulk_g2s(smem_addr(spb), a.spar + (size_t)t * a.spar_stride, (unsigned)sl.total, bar);
    }
  }
  if (MODE != MODE_FORCE)
    for (int q = lane; q < NACC; q += 32) acc[q] = T(0);
  chain_wait();
  if (IS_AF && lane == 0) {
    mbar_expect_tx(bar, (unsigned)sl.total);
    bulk_g2s(smem_addr(spb), a.spar + (size_t)t * a.spar_stride, (unsigned)sl.total, bar);
  }
  // what the preceding kernels produced for this atom, fetched while the copies are in flight
  const T* chrow = a.chan_in ? a.chan_in + gi * Fmax : nullptr;
  T fbx = T(0), fby = T(0), fbz = T(0);
  // dL/dF of one force component (the loss kernel's formula: Keras Huber(delta = 1) or squared error, mean)
  const T* fo_g = nullptr;
  const T* fl_g = nullptr;
  const T fscale = a.fscale;
  const bool hub = a.loss_kind == 0;
  auto fbar_of = [&](int q) -> T {
    const T e = fo_g[q] - fl_g[q];
    return fscale * (hub ? (e > T(1) ? T(1) : (e < T(-1) ? T(-1) : e)) : T(2) * e);
  };
  // dL/dW of this frame (virial loss of the energy + force + virial training, staf_model.py:313-384), kept behind
  // the group offsets
  T* wbs = reinterpret_cast<T*>(smem_raw + L.red) + 8;
  if (MODE == MODE_FGRAD) {
    fo_g = a.force + (size_t)b * a.nall * 3;
    fl_g = a.flab + (size_t)b * a.nall * 3;
    fbx = fbar_of(i * 3); fby = fbar_of(i * 3 + 1); fbz = fbar_of(i * 3 + 2);
    if (a.vacc) {
      // lane = slot: nine coalesced loads, nine warp sums
      double w = 0.0;
#pragma unroll
      for (int q = 0; q < 9; q++) {
        const double v = warp_sum(a.vacc[((size_t)b * 9 + q) * VIR_SLOTS + lane]);
        if (lane == q) w = v;
      }
      if (lane < 9) {
        const T e = (T)w - a.vlab[b * 9 + lane];
        wbs[lane] = a.vscale * (hub ? (e > T(1) ? T(1) : (e < T(-1) ? T(-1) : e)) : T(2) * e);
      }
    }
  }
  if (!mbar_wait(bar, 0)) {
    if (lane == 0) set_status(a.status, STAFB_ERR_STAGE_TIMEOUT);
    return;
  }
  int n = hdr[0];
  if (n > nr) n = nr;
  // first entry of every species' group (kept in shared memory like the counts, not in registers)
  if (lane == 0) {
    int o = 0;
    for (int q = 0; q < STAFB_MAX_TYPES; q++) {
      off[q] = o;
      o += (q < nt) ? hdr[2 + q] : 0;
    }
    off[STAFB_MAX_TYPES] = o;
  }
  __syncwarp();
  if (MODE == MODE_FGRAD) {
    // dF_k = Fbar_k - Fbar_i and its projection on the unit vector
    T4* dF = reinterpret_cast<T4*>(xtra);
    for (int k = lane; k < n; k += 32) {
      const int id = ids[k];
      const T4 u = U[k];
      T4 d;
      d.x = fbar_of(id * 3) - fbx; d.y = fbar_of(id * 3 + 1) - fby; d.z = fbar_of(id * 3 + 2) - fbz;
      if (a.vacc) {
        // W_ab = -sum f_a r_b over the pairs: the virial's cotangent shifts the neighbour's force cotangent by
        // -(dL/dW) r with r = r_i - r_k (grad_force/rad/reforce.cu.cc:165-234, grad_force/ang/reforce.cu.cc:274-446)
        const T r = T(1) / V[k].x;
        const T rx = u.x * r, ry = u.y * r, rz = u.z * r;
        d.x -= wbs[0] * rx + wbs[1] * ry + wbs[2] * rz;
        d.y -= wbs[3] * rx + wbs[4] * ry + wbs[5] * rz;
        d.z -= wbs[6] * rx + wbs[7] * ry + wbs[8] * rz;
      }
      d.w = d.x * u.x + d.y * u.y + d.z * u.z;
      dF[k] = d;
    }
  }
  if (MODE == MODE_FORCE) {
    // channel weights 0.25 * e3 * netderiv of every (class, channel pair); the 0.5 of E = 0.5 sum e and the 0.5 of
    // the symmetrised pair sum
    for (int idx = lane; idx < md.ncls * sl.maxp; idx += 32) {
      const int s = idx / sl.maxp, pr = idx - s * sl.maxp;
      T2 w = mk2(T(0), T(0));
      if (2 * pr < nact_s[s]) {
        const T2 ee = che_all[idx];
        w.x = T(0.25) * ee.x * chrow[Fr + actc[s * Famax + 2 * pr]];
        w.y = (2 * pr + 1 < nact_s[s]) ? T(0.25) * ee.y * chrow[Fr + actc[s * Famax + 2 * pr + 1]] : T(0);
      }
      wch_all[idx] = w;
    }
  }
  __syncwarp();

  T fix = T(0), fiy = T(0), fiz = T(0);  // FORCE: force on the central atom
  // ------------------------------------------------------------------ radial part
  if (MODE == MODE_FORCE) {
    // g_k = 0.5 * sum_c netderiv_c e2 e^{alpha d}(1 + alpha d) * dd/dr * u_k  (force/rad/reforce.cu.cc:45-136)
    for (int k = lane; k < nr; k += 32) {
      T gx = T(0), gy = T(0), gz = T(0);
      if (k < n) {
        int tk = 0;
#pragma unroll
        for (int q = 1; q < STAFB_MAX_TYPES; q++) tk += (q < nt && k >= off[q]) ? 1 : 0;
        const T4 u = U[k], v = V[k];
        const T dk = v.z;
        T w = T(0);
        for (int c = 0; c < Fr; c++) {
          const T4 rp = rpar[tk * Frmax + c];
          if (rp.z == T(0)) continue;
          w += chrow[c] * (T(0.5) * rp.z * Ex<T>::f(rp.x * dk) * (T(1) + rp.y * dk));
        }
        const T g = w * v.w;
        gx = g * u.x; gy = g * u.y; gz = g * u.z;
        fix -= gx; fiy -= gy; fiz -= gz;
      }
      xtra[k * 3 + 0] = gx; xtra[k * 3 + 1] = gy; xtra[k * 3 + 2] = gz;
    }
  } else {
    // one thread per (neighbour species q, channel c) walks that species' neighbours, so the sums over
    // neighbours need no cross-lane reduction; the per-species partial sums of a channel are combined
    // through rsum[].  AF, AFV: fingerprints; FGRAD: gradnet; all but AF: alpha2b terms.
    const int nqc = nt * Fr;
    for (int L0 = 0; L0 < nqc; L0 += 32) {
      const int Lq = L0 + lane;
      if (Lq < nqc) {
        const int q = Lq / Fr, c = Lq - q * Fr;
        const T4 rp = rpar[q * Frmax + c];
        T gn = T(0), ga = T(0);
        if (rp.z != T(0)) {
          const T als = rp.x, al = rp.y;
          const int r0_ = off[q], r1_ = off[q + 1];
          const T4* dF = reinterpret_cast<const T4*>(xtra);
#pragma unroll 4
          for (int r = r0_; r < r1_; r++) {
            const T4 v = V[r];
            const T dk = v.z;
            const T ex = Ex<T>::f(als * dk);
            if (MODE == MODE_FGRAD) {
              const T qq = T(0.5) * v.w * dF[r].w;
              gn += qq * ex * (T(1) + al * dk);
              ga += qq * ex * dk * (T(2) + al * dk);
            } else {
              gn += dk * ex;
              ga += ex * dk * dk;
            }
          }
          gn *= rp.z;
          ga *= (MODE == MODE_FGRAD ? chrow[c] : T(1)) * rp.z;
        }
        rsum[q * Frmax + c] = gn;
        if (MODE != MODE_AF) acc[ACC_A2 + q * Frmax + c] = ga;
      }
    }
    __syncwarp();
    for (int c = lane; c < Fr; c += 32) {
      T v = T(0);
      for (int q = 0; q < nt; q++) v += rsum[q * Frmax + c];
      a.out[gi * Fmax + c] = v;
    }
  }
  __syncwarp();

  // ------------------------------------------------------------------ angular part
  for (int ta = 0; ta < nt; ta++) {
    for (int tb = ta; tb < nt; tb++) {
      const int s = ta + tb;
      const int na_ = hdr[6 + ta], nb_ = hdr[6 + tb], oa = off[ta], ob = off[tb];
      const bool same = (ta == tb);
      const int np = same ? na_ * (na_ - 1) / 2 : na_ * nb_;
      if (np <= 0 || s >= md.ncls) continue;
      const int nact = nact_s[s];
      const int npair = (nact + 1) >> 1;
      for (int p0 = 0; p0 < npair; p0 += MAXP) {
        const int nchp = (npair - p0) < MAXP ? (npair - p0) : MAXP;
        const T4* chq = chq_all + s * sl.maxp + p0;
        const T4* chr = chr_all + s * sl.maxp + p0;
        // tables exp(a1*fc_k), exp(a2*fc_k) of the neighbours of the two species, all channel pairs of a
        // neighbour in flight together
        const int nu = same ? na_ : na_ + nb_;
        for (int r = lane; r < nu; r += 32) {
          const int k = (r < na_) ? oa + r : ob + (r - na_);
          const T fck = U[k].w * Ex<T>::scale();
          const T2 f2 = mk2(fck, fck);
#pragma unroll
          for (int lp = 0; lp < MAXP; lp++) {
            if (lp < nchp) {
              const T4 q = chq[lp];
              const T2 e1 = p_ex(p_mul(mk2(q.x, q.y), f2)), e2 = p_ex(p_mul(mk2(q.z, q.w), f2));
              T4 v;
              v.x = e1.x; v.y = e1.y; v.z = e2.x; v.w = e2.y;
              tab4[k * TSTR + lp] = v;
            }
          }
        }
        __syncwarp();
        if (MODE == MODE_FORCE) {
          const T2* wch = wch_all + s * sl.maxp + p0;
          const int npass = same ? 1 : 2;
          for (int pass = 0; pass < npass; pass++) {
            const int oo = pass == 0 ? oa : ob, op = pass == 0 ? ob : oa;
            const int no = pass == 0 ? na_ : nb_;
            const int npt = same ? na_ - 1 : (pass == 0 ? nb_ : na_);
            auto go = [&](auto tag) {
              constexpr int NCHP = decltype(tag)::value;
              if (same) pairs_force<T, NCHP, true>(U, V, tab4, chq, chr, wch, oo, op, no, npt, lane, xtra, fix, fiy, fiz);
              else pairs_force<T, NCHP, false>(U, V, tab4, chq, chr, wch, oo, op, no, npt, lane, xtra, fix, fiy, fiz);
            };
            switch (nchp) {
              case 1: go(std::integral_constant<int, 1>()); break;
              case 2: go(std::integral_constant<int, 2>()); break;
              case 3: go(std::integral_constant<int, 3>()); break;
              default: go(std::integral_constant<int, 4>()); break;
            }
          }
        } else {
          // per-lane sums, then the transposing butterfly: lane L ends up with the total of value index L (or
          // L >> 1, L >> 2 when fewer values are carried).  Value index = 8*lp + 4*h + v for channel 2*lp + h of
          // the chunk and term v (0 fingerprint / gradnet, 1..3 alpha1, alpha2, beta); AF carries v = 0 only,
          // index 2*lp + h.
          const T4* dF = reinterpret_cast<const T4*>(xtra);
          T tot = T(0);
          int vidx = -1;  // value index this lane holds after the reduction (-1: none)
          auto run = [&](auto nchp_tag) {
            constexpr int NCHP = decltype(nchp_tag)::value;
            T2 r0[NCHP], r1[NCHP], r2[NCHP], r3[NCHP];
            if (same) pairs_unordered<T, MODE, NCHP, true>(U, V, dF, tab4, nr, chq, chr, oa, ob, na_, nb_, lane, r0, r1, r2, r3);
            else pairs_unordered<T, MODE, NCHP, false>(U, V, dF, tab4, nr, chq, chr, oa, ob, na_, nb_, lane, r0, r1, r2, r3);
            if (MODE == MODE_AF) {
              constexpr int NV = NCHP == 1 ? 2 : (NCHP == 2 ? 4 : 8);
              T v[NV];
#pragma unroll
              for (int q = 0; q < NV; q++) v[q] = T(0);
#pragma unroll
              for (int lp = 0; lp < NCHP; lp++) { v[2 * lp] = r0[lp].x; v[2 * lp + 1] = r0[lp].y; }
              tot = multi_reduce<T, NV>(v, lane);
              constexpr int SH = NV == 2 ? 4 : (NV == 4 ? 3 : 2);  // log2(32 / NV)
              vidx = ((lane & ((1 << SH) - 1)) == 0) ? (lane >> SH) : -1;
              if (vidx >= 0) vidx = 8 * (vidx >> 1) + 4 * (vidx & 1);  // as (lp, h, v = 0)
            } else {
              constexpr int NV = NCHP == 1 ? 8 : (NCHP == 2 ? 16 : 32);
              T v[NV];
#pragma unroll
              for (int q = 0; q < NV; q++) v[q] = T(0);
#pragma unroll
              for (int lp = 0; lp < NCHP; lp++) {
                v[8 * lp] = r0[lp].x; v[8 * lp + 1] = r1[lp].x; v[8 * lp + 2] = r2[lp].x; v[8 * lp + 3] = r3[lp].x;
                v[8 * lp + 4] = r0[lp].y; v[8 * lp + 5] = r1[lp].y; v[8 * lp + 6] = r2[lp].y; v[8 * lp + 7] = r3[lp].y;
              }
              tot = multi_reduce<T, NV>(v, lane);
              constexpr int SH = NV == 8 ? 2 : (NV == 16 ? 1 : 0);
              vidx = ((lane & ((1 << SH) - 1)) == 0) ? (lane >> SH) : -1;
            }
          };
          switch (nchp) {
            case 1: run(std::integral_constant<int, 1>()); break;
            case 2: run(std::integral_constant<int, 2>()); break;
            case 3: run(std::integral_constant<int, 3>()); break;
            default: run(std::integral_constant<int, 4>()); break;
          }
          if (vidx >= 0) {
            const int lp = vidx >> 3, h = (vidx >> 2) & 1, v = vidx & 3;
            const int slot = 2 * (p0 + lp) + h;
            if (lp < nchp && slot < nact) {
              const int c = actc[s * Famax + slot];
              const T2 ee = che_all[s * sl.maxp + p0 + lp];
              const T cf = T(0.5) * (h ? ee.y : ee.x);
              if (v == 0) acc[ACC_GN + c] += cf * tot;
              else if (MODE != MODE_AF) {
                const T hn = MODE == MODE_FGRAD ? cf * chrow[Fr + c] : cf;
                acc[ACC_A3 + (s * Famax + c) * 3 + (v - 1)] += hn * tot;
              }
            }
          }
        }
        __syncwarp();  // the next chunk rewrites the tables
      }
    }
  }
  __syncwarp();

  // ------------------------------------------------------------------ write-back
  if (IS_AF) {
    for (int c = lane; c < Fa; c += 32) a.out[gi * Fmax + Fr + c] = acc[ACC_GN + c];
    for (int c = Fr + Fa + lane; c < Fmax; c += 32) a.out[gi * Fmax + c] = T(0);
    if (MODE == MODE_AFV) {
      T* vr = a.vout + gi * a.nv;
      for (int q = lane; q < a.nv; q += 32) vr[q] = acc[q];
    }
  } else if (MODE == MODE_FORCE) {
    T* fbo = a.out + (size_t)b * a.nall * 3;
    for (int q = lane; q < 3 * n; q += 32) atomicAdd(fbo + (size_t)ids[q / 3] * 3 + (q % 3), xtra[q]);
    fix = warp_sum(fix); fiy = warp_sum(fiy); fiz = warp_sum(fiz);
    if (lane == 0) {
      atomicAdd(fbo + (size_t)i * 3 + 0, fix);
      atomicAdd(fbo + (size_t)i * 3 + 1, fiy);
      atomicAdd(fbo + (size_t)i * 3 + 2, fiz);
    }
    if (VIR) {
      // W_ab -= g_a * r_b with g the force this centre puts on neighbour k and r = r_i - r_k
      // (force/rad/reforce.cu.cc:174-287, force/ang/reforce.cu.cc:269-457 of the reference)
      // one row of W at a time keeps the epilogue's register footprint below the main loop's
#pragma unroll 1
      for (int c = 0; c < 3; c++) {
        T w0 = T(0), w1 = T(0), w2 = T(0);
        for (int k = lane; k < n; k += 32) {
          const T4 u = U[k];
          const T g = xtra[k * 3 + c] / V[k].x;  // g_a * |r|
          w0 -= g * u.x; w1 -= g * u.y; w2 -= g * u.z;
        }
        w0 = warp_sum(w0); w1 = warp_sum(w1); w2 = warp_sum(w2);
        if (lane == 0) {
          double* vs = a.vir + ((size_t)b * 9 + c * 3) * VIR_SLOTS + (i & (VIR_SLOTS - 1));
          atomicAdd(vs, (double)w0);
          atomicAdd(vs + VIR_SLOTS, (double)w1);
          atomicAdd(vs + 2 * VIR_SLOTS, (double)w2);
        }
      }
    }
  } else {  // FGRAD
    for (int c = lane; c < Fa; c += 32) a.out[gi * Fmax + Fr + c] = acc[ACC_GN + c];
    for (int c = Fr + Fa + lane; c < Fmax; c += 32) a.out[gi * Fmax + c] = T(0);
    if (a.grad) {
      T* g2 = a.grad + md.off_a2[t];
      for (int q = lane; q < nt * Fr; q += 32) {
        const T v = acc[ACC_A2 + (q / Fr) * Frmax + (q % Fr)];
        if (v != T(0)) atomicAdd(g2 + q, v);
      }
      T* g3 = a.grad + md.off_a3[t];
      for (int q = lane; q < md.C * 3 * Fa; q += 32) {
        const int sc = q / 3, comp = q - sc * 3, s = sc / Fa, c = sc - s * Fa;
        const T v = acc[ACC_A3 + (s * Famax + c) * 3 + comp];
        if (v != T(0)) atomicAdd(g3 + q, v);
      }
    }
  }
}
