// Fused energy/force/training path: descriptors never leave the chip.
//
// The operator path (ops.cu) has to honour the reference's tensor contract, which pushes
// ~110 KB per atom of angular descriptors (angdescr, intmap3b, der3b) through HBM.  Here the
// neighbour kernel leaves only a compact sorted neighbour row per atom (MIC vector, radial
// descriptor, cutoff, their scalar derivatives: ~2 KB) and every sweep rebuilds the triplet
// geometry in registers from rows staged in shared memory.  One warp owns one central atom.
//
// Triplets are enumerated per species-pair class (ta <= tb) rather than in the reference's
// j<k slot order: inside a class every triplet uses the same parameter row
// (row = type_j + type_k, STAF/src/fingerprint/ang/reforce.cu.cc:56), so the channel loop is
// uniform across the warp and channels whose squared embedding is zero are skipped for the
// whole class.  exp(a1*sj + a2*sk) is formed as a product of per-neighbour factors
// exp(a1*sj), exp(a2*sk) tabulated once per (class, channel chunk).
//
// Math: STAF/src/fingerprint, force, grad_finger, grad_force (rad and ang) reforce.cu.cc and
// STAF/staf_models/staf_model.py:168-258 of the reference (see include/stafb.h).
#include <math.h>
#include <stdlib.h>
#include <string.h>
#include "common.cuh"

namespace stafb {

constexpr int MAXCH = 8;    // channels processed per pair sweep
constexpr int SW_WARPS = 4; // warps (= atoms) per block in the sweep kernels
constexpr int ML_WARPS = 8; // atoms per block in the MLP kernels

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

template <class T>
struct SweepIn {
  const T* geom;   // [nf,N,nr,4]
  const T* gsc;    // [nf,N,nr,2]
  const T* rad;    // [nf,N,nr]
  const T* d3s;    // [nf,N,nr]
  const int* im2;  // [nf,N,nr+1]
  const int* ntr;  // [nf,N]
  int nf, nr;
};

enum { MODE_AF = 0, MODE_FORCE = 1, MODE_FGRAD = 2, MODE_AFGRAD = 3 };

// species-major enumeration: block -> (species, first atom); W atoms per block
__device__ __forceinline__ bool locate_atom(const ModelDev& md, int nf, int W, int warp, int& t, int& b, int& i) {
  int blk = blockIdx.x;
  t = 0;
  while (t < md.nt - 1) {
    const int nb = (nf * md.tipos[t] + W - 1) / W;
    if (blk < nb) break;
    blk -= nb;
    t++;
  }
  const int q = blk * W + warp;
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

// per-warp shared memory layout of the sweep kernels (offsets in bytes)
struct SweepLayout {
  int u, d, fc, gd, gfc, tab, chp, xtra, acc, ids, tj, lst, actl, total;
};

template <class T>
static inline SweepLayout sweep_layout(int nr, int nt, int xt, int nacc, int famax) {
  SweepLayout L;
  int o = 0;
  auto take = [&](int bytes) { int r = o; o += (bytes + 15) & ~15; return r; };
  L.u = take(nr * 4 * sizeof(T));
  L.d = take(nr * sizeof(T));
  L.fc = take(nr * sizeof(T));
  L.gd = take(nr * sizeof(T));
  L.gfc = take(nr * sizeof(T));
  L.tab = take(MAXCH * nr * 2 * sizeof(T));
  L.chp = take(MAXCH * 8 * sizeof(T));
  L.xtra = take(nr * xt * sizeof(T));
  L.acc = take(nacc * sizeof(T));
  L.ids = take(nr * sizeof(int));
  L.tj = take(nr);
  L.lst = take(nt * nr);
  L.actl = take(famax);
  L.total = o;
  return L;
}

template <class T, int MODE>
__global__ void __launch_bounds__(SW_WARPS * 32)
    k_sweep(ModelDev md, SweepIn<T> in, SweepLayout L, const T* __restrict__ theta, const T* __restrict__ emb,
            const T* __restrict__ chan_in,  // FORCE/FGRAD: netderiv[nf,N,Fmax]; AFGRAD: dL/dAF[nf,N,Fmax]
            const T* __restrict__ fbar,     // FGRAD: dL/dF[nf,3N]
            T* __restrict__ out,            // AF: af[nf,N,Fmax]; FORCE: force[nf,3N]; FGRAD: gradnet[nf,N,Fmax]
            T* __restrict__ grad) {         // FGRAD/AFGRAD: flat parameter gradient (accumulated)
  extern __shared__ __align__(16) unsigned char smem_raw[];
  typedef typename Vec4<T>::type T4;
  typedef typename Vec2<T>::type T2;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int t, b, i;
  if (!locate_atom(md, in.nf, SW_WARPS, warp, t, b, i)) return;
  unsigned char* base = smem_raw + (size_t)warp * L.total;
  T4* u = reinterpret_cast<T4*>(base + L.u);
  T* d = reinterpret_cast<T*>(base + L.d);
  T* fc = reinterpret_cast<T*>(base + L.fc);
  T* gd = reinterpret_cast<T*>(base + L.gd);
  T* gfc = reinterpret_cast<T*>(base + L.gfc);
  T2* tab = reinterpret_cast<T2*>(base + L.tab);
  T* chp = reinterpret_cast<T*>(base + L.chp);
  T* xtra = reinterpret_cast<T*>(base + L.xtra);
  T* acc = reinterpret_cast<T*>(base + L.acc);
  int* ids = reinterpret_cast<int*>(base + L.ids);
  unsigned char* tj = base + L.tj;
  unsigned char* lst = base + L.lst;
  unsigned char* actl = base + L.actl;

  const int N = md.N, nr = in.nr, nt = md.nt;
  const int Fr = md.Fr[t], Fa = md.Fa[t], Fmax = md.Fmax;
  const size_t gi = (size_t)b * N + i;
  const T* a2 = theta + md.off_a2[t];
  const T* a3 = theta + md.off_a3[t];
  const T* e2 = emb + md.off_emb[t];
  const T* e3 = e2 + nt * Fr;
  const T* chrow = chan_in ? chan_in + gi * Fmax : nullptr;
  // accumulator regions inside acc[]
  const int ACC_GN = 0;                      // [Famax]     AF: fingerprints; FGRAD: gradnet (angular part)
  const int ACC_A2 = md.Famax;               // [nt*Frmax]  dL/dalpha2b
  const int ACC_A3 = ACC_A2 + nt * md.Frmax; // [C*3*Famax] dL/dalpha3b
  const int NACC = ACC_A3 + md.C * 3 * md.Famax;

  int n = in.im2[gi * (nr + 1)];
  if (n > nr) n = nr;
  int m = in.ntr[gi];
  if (m > n) m = n;
  for (int k = lane; k < n; k += 32) {
    T4 g = reinterpret_cast<const T4*>(in.geom)[gi * nr + k];
    const T inv = T(1) / g.w;
    T4 q;
    q.x = g.x * inv; q.y = g.y * inv; q.z = g.z * inv; q.w = g.w;
    u[k] = q;
    d[k] = in.rad[gi * nr + k];
    fc[k] = in.d3s[gi * nr + k];
    T2 s = reinterpret_cast<const T2*>(in.gsc)[gi * nr + k];
    gd[k] = s.x;
    gfc[k] = s.y;
    const int id = in.im2[gi * (nr + 1) + 1 + k];
    ids[k] = id;
    tj[k] = (unsigned char)md.type_of(id);
  }
  if (MODE != MODE_FORCE)
    for (int q = lane; q < NACC; q += 32) acc[q] = T(0);
  __syncwarp();
  // per-species lists of the angular neighbours (first m sorted entries)
  int cnt[STAFB_MAX_TYPES];
  const unsigned lt = (1u << lane) - 1u;
#pragma unroll
  for (int t2 = 0; t2 < STAFB_MAX_TYPES; t2++) {
    cnt[t2] = 0;
    if (t2 < nt) {
      for (int k0 = 0; k0 < m; k0 += 32) {
        const int k = k0 + lane;
        const bool p = (k < m) && (tj[k] == t2);
        const unsigned bal = __ballot_sync(0xffffffffu, p);
        if (p) lst[t2 * nr + cnt[t2] + __popc(bal & lt)] = (unsigned char)k;
        cnt[t2] += __popc(bal);
      }
    }
  }
  T fix = T(0), fiy = T(0), fiz = T(0);  // FORCE: force on the central atom
  if (MODE == MODE_FORCE) {
    for (int q = lane; q < 3 * nr; q += 32) xtra[q] = T(0);
  }
  if (MODE == MODE_FGRAD) {
    // dF_k = Fbar_k - Fbar_i and its projection on the unit vector
    const T* fb = fbar + (size_t)b * N * 3;
    const T fx = fb[i * 3], fy = fb[i * 3 + 1], fz = fb[i * 3 + 2];
    for (int k = lane; k < n; k += 32) {
      const int id = ids[k];
      const T dx = fb[id * 3] - fx, dy = fb[id * 3 + 1] - fy, dz = fb[id * 3 + 2] - fz;
      xtra[k * 4 + 0] = dx; xtra[k * 4 + 1] = dy; xtra[k * 4 + 2] = dz;
      xtra[k * 4 + 3] = dx * u[k].x + dy * u[k].y + dz * u[k].z;
    }
  }
  __syncwarp();

  // ------------------------------------------------------------------ radial part
  if (MODE == MODE_AF) {
    for (int c = 0; c < Fr; c++) {
      T s = T(0);
      for (int k = lane; k < n; k += 32) {
        const T ch = e2[Fr * tj[k] + c];
        if (ch != T(0)) s += d[k] * (r_exp(a2[Fr * tj[k] + c] * d[k]) * ch);
      }
      s = warp_sum(s);
      if (lane == 0) out[gi * Fmax + c] = s;
    }
  } else if (MODE == MODE_FORCE) {
    for (int k = lane; k < n; k += 32) {
      const int tk = tj[k];
      const T dk = d[k];
      T w = T(0);
      for (int c = 0; c < Fr; c++) {
        const T ch = e2[Fr * tk + c];
        if (ch == T(0)) continue;
        const T al = a2[Fr * tk + c];
        w += chrow[c] * (T(0.5) * ch * r_exp(al * dk) * (T(1) + al * dk));
      }
      const T g = w * gd[k];
      const T gx = g * u[k].x, gy = g * u[k].y, gz = g * u[k].z;
      xtra[k * 3 + 0] = gx; xtra[k * 3 + 1] = gy; xtra[k * 3 + 2] = gz;
      fix -= gx; fiy -= gy; fiz -= gz;
    }
  } else {  // FGRAD / AFGRAD: gradients with respect to alpha2b (and gradnet for FGRAD)
    for (int c = 0; c < Fr; c++) {
      const T cin = chrow[c];  // FGRAD: netderiv ; AFGRAD: dL/dAF
      T gn = T(0);
      T ga[STAFB_MAX_TYPES];
#pragma unroll
      for (int q = 0; q < STAFB_MAX_TYPES; q++) ga[q] = T(0);
      for (int k = lane; k < n; k += 32) {
        const int tk = tj[k];
        const T ch = e2[Fr * tk + c];
        if (ch == T(0)) continue;
        const T al = a2[Fr * tk + c], dk = d[k];
        const T ex = r_exp(al * dk);
        T va;
        if (MODE == MODE_FGRAD) {
          const T q = T(0.5) * gd[k] * xtra[k * 4 + 3];
          gn += q * ch * ex * (T(1) + al * dk);
          va = q * cin * ch * ex * dk * (T(2) + al * dk);
        } else {
          va = cin * ch * ex * dk * dk;
        }
#pragma unroll
        for (int q = 0; q < STAFB_MAX_TYPES; q++)
          if (q == tk) ga[q] += va;
      }
      if (MODE == MODE_FGRAD) {
        gn = warp_sum(gn);
        if (lane == 0) out[gi * Fmax + c] = gn;
      }
#pragma unroll
      for (int q = 0; q < STAFB_MAX_TYPES; q++) {
        if (q < nt) {
          const T s = warp_sum(ga[q]);
          if (lane == 0) acc[ACC_A2 + q * md.Frmax + c] += s;
        }
      }
    }
  }
  __syncwarp();

  // ------------------------------------------------------------------ angular part
  for (int ta = 0; ta < nt; ta++) {
    for (int tb = ta; tb < nt; tb++) {
      const int s = ta + tb;
      int na_ = 0, nb_ = 0;
#pragma unroll
      for (int q = 0; q < STAFB_MAX_TYPES; q++) {
        if (q == ta) na_ = cnt[q];
        if (q == tb) nb_ = cnt[q];
      }
      const int np = (ta == tb) ? na_ * (na_ - 1) / 2 : na_ * nb_;
      if (np <= 0 || s >= md.ncls) continue;
      const unsigned char* la = lst + ta * nr;
      const unsigned char* lb = lst + tb * nr;
      // active channels of this class
      int nact = 0;
      for (int c0 = 0; c0 < Fa; c0 += 32) {
        const int c = c0 + lane;
        const bool p = (c < Fa) && (e3[s * Fa + c] != T(0));
        const unsigned bal = __ballot_sync(0xffffffffu, p);
        if (p) actl[nact + __popc(bal & lt)] = (unsigned char)c;
        nact += __popc(bal);
      }
      __syncwarp();
      for (int c0 = 0; c0 < nact; c0 += MAXCH) {
        const int nch = (nact - c0) < MAXCH ? (nact - c0) : MAXCH;
        if (lane < nch) {
          const int c = actl[c0 + lane];
          const T* al = a3 + (s * Fa + c) * 3;
          const T ee = e3[s * Fa + c];
          chp[lane * 8 + 0] = al[0];
          chp[lane * 8 + 1] = al[1];
          chp[lane * 8 + 2] = al[2];
          if (MODE == MODE_AF) chp[lane * 8 + 3] = T(0.5) * ee;
          if (MODE == MODE_FORCE) chp[lane * 8 + 3] = T(0.5) * chrow[Fr + c] * ee;
          if (MODE == MODE_FGRAD) { chp[lane * 8 + 3] = T(0.5) * ee; chp[lane * 8 + 4] = chrow[Fr + c]; }
          if (MODE == MODE_AFGRAD) chp[lane * 8 + 3] = T(0.5) * chrow[Fr + c] * ee;
        }
        __syncwarp();
        // tables exp(a1*fc_k), exp(a2*fc_k) for the neighbours of the two species
        const int nu = (ta == tb) ? na_ : na_ + nb_;
        for (int q = lane; q < nch * nu; q += 32) {
          const int l = q / nu, r = q - l * nu;
          const int k = (r < na_) ? la[r] : lb[r - na_];
          T2 v;
          v.x = r_exp(chp[l * 8 + 0] * fc[k]);
          v.y = r_exp(chp[l * 8 + 1] * fc[k]);
          tab[l * nr + k] = v;
        }
        __syncwarp();
        T r0[MAXCH], r1[MAXCH], r2[MAXCH], r3[MAXCH];
#pragma unroll
        for (int l = 0; l < MAXCH; l++) r0[l] = r1[l] = r2[l] = r3[l] = T(0);
        for (int p = lane; p < np; p += 32) {
          int ja, kb;
          if (ta == tb) unrank_pair(p, na_, ja, kb);
          else { ja = p / nb_; kb = p - ja * nb_; }
          const int j = la[ja], k = lb[kb];
          const T4 uj = u[j], uk = u[k];
          const T fcj = fc[j], fck = fc[k];
          const T cs = uj.x * uk.x + uj.y * uk.y + uj.z * uk.z;
          const T half = T(0.5) * (cs + T(1));
          const T tt = half * fcj * fck;
          T Q = T(0), Pj = T(0), Pk = T(0);
          if (MODE == MODE_FGRAD) {
            const T hf = T(0.5) * fcj * fck;
            const T ajk = hf / uj.w, akj = hf / uk.w;
            const T bjk = -cs * ajk + half * gfc[j] * fck;
            const T bkj = -cs * akj + half * gfc[k] * fcj;
            const T* dFj = xtra + j * 4;
            const T* dFk = xtra + k * 4;
            const T djuk = dFj[0] * uk.x + dFj[1] * uk.y + dFj[2] * uk.z;
            const T dkuj = dFk[0] * uj.x + dFk[1] * uj.y + dFk[2] * uj.z;
            Q = ajk * djuk + bjk * dFj[3] + akj * dkuj + bkj * dFk[3];
            Pj = gfc[j] * dFj[3];
            Pk = gfc[k] * dFk[3];
          }
          T D = T(0), BJ = T(0), BK = T(0);
          const T sj = fcj, sk = fck;
#pragma unroll
          for (int l = 0; l < MAXCH; l++) {
            if (l < nch) {
              const T2 A = tab[l * nr + j], B = tab[l * nr + k];
              const T al1 = chp[l * 8 + 0], al2 = chp[l * 8 + 1], be = chp[l * 8 + 2], cf = chp[l * 8 + 3];
              const T S1 = A.y * B.x;  // exp(a2*sj + a1*sk)
              const T S2 = A.x * B.y;  // exp(a1*sj + a2*sk)
              const T eb = r_exp(be * tt);
              if (MODE == MODE_AF) {
                r0[l] += cf * tt * (S1 + S2) * eb;
              } else if (MODE == MODE_FORCE) {
                D += cf * (eb * (T(1) + be * tt) * (S1 + S2) * T(0.5));
                BJ += cf * ((al1 * S2 + al2 * S1) * eb * T(0.5) * tt);
                BK += cf * ((al1 * S1 + al2 * S2) * eb * T(0.5) * tt);
              } else if (MODE == MODE_AFGRAD) {
                const T cm = cf * eb * tt;
                r1[l] += cm * (S2 * sj + S1 * sk);
                r2[l] += cm * (S2 * sk + S1 * sj);
                r3[l] += cm * (S1 + S2) * tt;
              } else {  // FGRAD
                const T NG = chp[l * 8 + 4];
                const T ss = S1 + S2, opb = T(1) + be * tt;
                const T delta = eb * opb * ss * T(0.5);
                const T et = eb * T(0.5) * tt;
                const T Bj = (al1 * S2 + al2 * S1) * et, Bk = (al1 * S1 + al2 * S2) * et;
                r0[l] += cf * (delta * Q + Bj * Pj + Bk * Pk);
                const T hn = cf * NG;
                const T ba1 = eb * opb * (S1 * sk + S2 * sj) * T(0.5);
                const T ba2 = eb * opb * (S1 * sj + S2 * sk) * T(0.5);
                const T bb = eb * tt * (T(2) + be * tt) * ss * T(0.5);
                const T a1j = (S2 + al1 * S2 * sj + al2 * S1 * sk) * et;
                const T a2j = (S1 + al2 * S1 * sj + al1 * S2 * sk) * et;
                const T a1k = (S1 + al1 * S1 * sk + al2 * S2 * sj) * et;
                const T a2k = (S2 + al2 * S2 * sk + al1 * S1 * sj) * et;
                r1[l] += hn * (ba1 * Q + a1j * Pj + a1k * Pk);
                r2[l] += hn * (ba2 * Q + a2j * Pj + a2k * Pk);
                r3[l] += hn * (bb * Q + Bj * tt * Pj + Bk * tt * Pk);
              }
            }
          }
          if (MODE == MODE_FORCE) {
            const T hf = T(0.5) * fcj * fck;
            const T ajk = hf / uj.w, akj = hf / uk.w;
            const T bjk = -cs * ajk + half * gfc[j] * fck;
            const T bkj = -cs * akj + half * gfc[k] * fcj;
            // f_ij = D*(ajk*uk + bjk*uj) + BJ*gfc_j*uj ; f_ik likewise
            const T cjk = D * ajk, cjj = D * bjk + BJ * gfc[j];
            const T ckj = D * akj, ckk = D * bkj + BK * gfc[k];
            const T fjx = cjk * uk.x + cjj * uj.x, fjy = cjk * uk.y + cjj * uj.y, fjz = cjk * uk.z + cjj * uj.z;
            const T fkx = ckj * uj.x + ckk * uk.x, fky = ckj * uj.y + ckk * uk.y, fkz = ckj * uj.z + ckk * uk.z;
            atomicAdd(&xtra[j * 3 + 0], fjx);
            atomicAdd(&xtra[j * 3 + 1], fjy);
            atomicAdd(&xtra[j * 3 + 2], fjz);
            atomicAdd(&xtra[k * 3 + 0], fkx);
            atomicAdd(&xtra[k * 3 + 1], fky);
            atomicAdd(&xtra[k * 3 + 2], fkz);
            fix -= fjx + fkx;
            fiy -= fjy + fky;
            fiz -= fjz + fkz;
          }
        }
        if (MODE != MODE_FORCE) {
#pragma unroll
          for (int l = 0; l < MAXCH; l++) {
            if (l < nch) {
              const int c = actl[c0 + l];
              if (MODE == MODE_AF || MODE == MODE_FGRAD) {
                const T v = warp_sum(r0[l]);
                if (lane == 0) acc[ACC_GN + c] += v;
              }
              if (MODE == MODE_AFGRAD || MODE == MODE_FGRAD) {
                const T v1 = warp_sum(r1[l]), v2 = warp_sum(r2[l]), v3 = warp_sum(r3[l]);
                if (lane == 0) {
                  T* g = acc + ACC_A3 + (s * md.Famax + c) * 3;
                  g[0] += v1; g[1] += v2; g[2] += v3;
                }
              }
            }
          }
        }
        __syncwarp();
      }
    }
  }
  __syncwarp();

  // ------------------------------------------------------------------ write-back
  if (MODE == MODE_AF) {
    for (int c = lane; c < Fa; c += 32) out[gi * Fmax + Fr + c] = acc[ACC_GN + c];
    for (int c = Fr + Fa + lane; c < Fmax; c += 32) out[gi * Fmax + c] = T(0);
  } else if (MODE == MODE_FORCE) {
    T* fb = out + (size_t)b * N * 3;
    for (int q = lane; q < 3 * n; q += 32) atomicAdd(fb + (size_t)ids[q / 3] * 3 + (q % 3), xtra[q]);
    fix = warp_sum(fix); fiy = warp_sum(fiy); fiz = warp_sum(fiz);
    if (lane == 0) {
      atomicAdd(fb + (size_t)i * 3 + 0, fix);
      atomicAdd(fb + (size_t)i * 3 + 1, fiy);
      atomicAdd(fb + (size_t)i * 3 + 2, fiz);
    }
  } else {
    if (MODE == MODE_FGRAD) {
      for (int c = lane; c < Fa; c += 32) out[gi * Fmax + Fr + c] = acc[ACC_GN + c];
      for (int c = Fr + Fa + lane; c < Fmax; c += 32) out[gi * Fmax + c] = T(0);
    }
    T* g2 = grad + md.off_a2[t];
    for (int q = lane; q < nt * Fr; q += 32) {
      const T v = acc[ACC_A2 + (q / Fr) * md.Frmax + (q % Fr)];
      if (v != T(0)) atomicAdd(g2 + q, v);
    }
    T* g3 = grad + md.off_a3[t];
    for (int q = lane; q < md.C * 3 * Fa; q += 32) {
      const int sc = q / 3, comp = q - sc * 3, s = sc / Fa, c = sc - s * Fa;
      const T v = acc[ACC_A3 + (s * md.Famax + c) * 3 + comp];
      if (v != T(0)) atomicAdd(g3 + q, v);
    }
  }
}

// ---------------------------------------------------------------------------- MLP head
// x = log(AF+1e-3) - mu ; Dense(tanh)... Dense(1)  (staf_models/staf_model.py:188-191,
// libstaf/src/mlp/staf_mlp_ort.cc:196-242).  One warp per atom; weights stream through L1/L2.
template <class T>
__device__ __forceinline__ void mlp_forward(const ModelDev& md, int t, int lane, const T* __restrict__ w,
                                            const T* x, T* h /*[Hsum]*/) {
  const int Lq = md.n_dense;
  const T* hin = x;
  for (int l = 0; l < Lq; l++) {
    const int in = md.in_of(t, l), out = md.width[l];
    const T* Wl = w + md.w_off(t, l);
    const T* Bl = Wl + in * out;
    T* hout = h + md.h_off(l);
    for (int j = lane; j < out; j += 32) {
      T s = Bl[j];
      for (int q = 0; q < in; q++) s += hin[q] * Wl[q * out + j];
      if (l < Lq - 1) s = r_tanh(s);
      hout[j] = s;
    }
    __syncwarp();
    hin = hout;
  }
}

// y[i] = sum_j v[j] * W[i,j]  for i < in (row-major [in,out]); coalesced over j, reduced per row
template <class T>
__device__ __forceinline__ void matvec_t(int lane, const T* __restrict__ Wl, int in, int out, const T* v, T* y) {
  for (int q = 0; q < in; q++) {
    T s = T(0);
    for (int j = lane; j < out; j += 32) s += v[j] * Wl[q * out + j];
    s = warp_sum(s);
    if (lane == 0) y[q] = s;
  }
  __syncwarp();
}

template <class T>
__global__ void __launch_bounds__(ML_WARPS * 32)
    k_mlp_fwd(ModelDev md, int nf, const T* __restrict__ theta, const T* __restrict__ af, T* __restrict__ acts,
              T* __restrict__ e_atom, T* __restrict__ netderiv) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int t, b, i;
  if (!locate_atom(md, nf, ML_WARPS, warp, t, b, i)) return;
  const int per = md.Fmax + md.Hsum + 2 * md.maxw;
  T* x = reinterpret_cast<T*>(smem_raw) + (size_t)warp * per;
  T* h = x + md.Fmax;
  T* p0 = h + md.Hsum;
  T* p1 = p0 + md.maxw;
  const int F = md.Fr[t] + md.Fa[t], Lq = md.n_dense;
  const size_t gi = (size_t)b * md.N + i;
  const T* mu = theta + md.off_mu[t];
  const T* w = theta + md.off_w[t];
  for (int q = lane; q < F; q += 32) x[q] = r_log(af[gi * md.Fmax + q] + T(1e-3)) - mu[q];
  __syncwarp();
  mlp_forward(md, t, lane, w, x, h);
  for (int q = lane; q < md.Hsum; q += 32) acts[gi * md.Hsum + q] = h[q];
  if (lane == 0) e_atom[gi] = h[md.h_off(Lq - 1)];
  // de/dx by the reverse sweep
  T* pn = p0;  // cotangent on the output of layer l
  T* pc = p1;
  if (lane == 0) pn[0] = T(1);
  __syncwarp();
  for (int l = Lq - 1; l >= 0; l--) {
    const int in = md.in_of(t, l), out = md.width[l];
    if (l < Lq - 1) {
      const T* hl = h + md.h_off(l);
      for (int j = lane; j < out; j += 32) pn[j] *= (T(1) - hl[j] * hl[j]);
      __syncwarp();
    }
    matvec_t(lane, w + md.w_off(t, l), in, out, pn, pc);
    T* tmp = pn; pn = pc; pc = tmp;
  }
  for (int q = lane; q < md.Fmax; q += 32)
    netderiv[gi * md.Fmax + q] = (q < F) ? pn[q] / (af[gi * md.Fmax + q] + T(1e-3)) : T(0);
}

// Backward of  S = sum_a ebar[a]*e[a] + sum_{a,c} u[a,c]*netderiv[a,c]  with respect to the
// weights, mu and AF: the first term is plain back-propagation, the second is the derivative
// of a directional derivative (tangent v = u/(AF+eps) pushed forward, then reversed) - what
// TensorFlow's autodiff does through grad_ene for the force loss (staf_model.py:191,225-228).
template <class T>
__global__ void __launch_bounds__(ML_WARPS * 32)
    k_mlp_bwd(ModelDev md, int nf, const T* __restrict__ theta, const T* __restrict__ af,
              const T* __restrict__ acts, const T* __restrict__ ebar /*[nf]*/, const T* __restrict__ u /*[nf,N,Fmax]*/,
              T* __restrict__ gaf, T* __restrict__ grad) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int t, b, i;
  const bool active = locate_atom(md, nf, ML_WARPS, warp, t, b, i);
  // locate_atom leaves t valid for the whole block (blocks are species-homogeneous)
  const int Fm = md.Fmax, Hs = md.Hsum, mw = md.maxw;
  const int per = 3 * Fm + 5 * Hs + 2 * mw;
  T* x = reinterpret_cast<T*>(smem_raw) + (size_t)warp * per;
  T* v = x + Fm;      // tangent on x
  T* q0 = v + Fm;     // dS/dx
  T* h = q0 + Fm;     // activations (outputs of every Dense)
  T* hd = h + Hs;     // tangents of the activations
  T* ad = hd + Hs;    // tangents of the pre-activations
  T* dq = ad + Hs;    // cotangent on the pre-activation (first-order channel)
  T* dp = dq + Hs;    // cotangent on the pre-activation tangent
  T* c0 = dp + Hs;    // scratch [maxw]
  T* c1 = c0 + mw;
  const int F = md.Fr[t] + md.Fa[t], Lq = md.n_dense;
  const T* w = theta + md.off_w[t];
  const size_t gi = active ? (size_t)b * md.N + i : 0;
  if (active) {
    const T* mu = theta + md.off_mu[t];
    for (int q = lane; q < F; q += 32) {
      const T den = af[gi * Fm + q] + T(1e-3);
      x[q] = r_log(den) - mu[q];
      v[q] = u[gi * Fm + q] / den;
    }
    for (int q = lane; q < Hs; q += 32) h[q] = acts[gi * Hs + q];
    __syncwarp();
    // forward tangent
    const T* hdin = v;
    for (int l = 0; l < Lq; l++) {
      const int in = md.in_of(t, l), out = md.width[l];
      const T* Wl = w + md.w_off(t, l);
      T* ho = h + md.h_off(l);
      T* hdo = hd + md.h_off(l);
      T* ado = ad + md.h_off(l);
      for (int j = lane; j < out; j += 32) {
        T s = T(0);
        for (int q = 0; q < in; q++) s += hdin[q] * Wl[q * out + j];
        ado[j] = s;
        hdo[j] = (l < Lq - 1) ? s * (T(1) - ho[j] * ho[j]) : s;
      }
      __syncwarp();
      hdin = hdo;
    }
    // reverse over (h, hd): cq = cotangent on h[l+1], cp = cotangent on hd[l+1]
    T* cq = c0;
    T* cp = c1;
    if (lane == 0) { cq[0] = ebar[b]; cp[0] = T(1); }
    __syncwarp();
    for (int l = Lq - 1; l >= 0; l--) {
      const int in = md.in_of(t, l), out = md.width[l];
      const T* Wl = w + md.w_off(t, l);
      const T* ho = h + md.h_off(l);
      const T* ado = ad + md.h_off(l);
      T* dql = dq + md.h_off(l);
      T* dpl = dp + md.h_off(l);
      for (int j = lane; j < out; j += 32) {
        T qa, pa;
        if (l < Lq - 1) {
          const T hh = ho[j], d1 = T(1) - hh * hh;
          pa = cp[j] * d1;
          qa = cq[j] * d1 + cp[j] * (T(-2) * hh * d1 * ado[j]);
        } else {
          pa = cp[j];
          qa = cq[j];
        }
        dql[j] = qa;
        dpl[j] = pa;
      }
      __syncwarp();
      // propagate to the layer input: cq_in = W dq, cp_in = W dp  (reuse cq/cp as outputs)
      for (int q = 0; q < in; q++) {
        T s1 = T(0), s2 = T(0);
        for (int j = lane; j < out; j += 32) {
          const T wv = Wl[q * out + j];
          s1 += dql[j] * wv;
          s2 += dpl[j] * wv;
        }
        s1 = warp_sum(s1);
        s2 = warp_sum(s2);
        if (lane == 0) {
          if (l == 0) { q0[q] = s1; c1[q] = s2; }  // dS/dx, dS/dv
          else { cq[q] = s1; cp[q] = s2; }
        }
      }
      __syncwarp();
    }
    // dS/dAF: through x = log(AF+eps) - mu and through v = u/(AF+eps)
    for (int q = lane; q < Fm; q += 32) {
      T g = T(0);
      if (q < F) {
        const T den = af[gi * Fm + q] + T(1e-3);
        g = q0[q] / den + c1[q] * (-u[gi * Fm + q] / (den * den));
      }
      gaf[gi * Fm + q] = g;
    }
  } else {
    for (int q = lane; q < Fm; q += 32) { x[q] = T(0); v[q] = T(0); q0[q] = T(0); }
    for (int q = lane; q < Hs; q += 32) { h[q] = hd[q] = dq[q] = dp[q] = T(0); }
  }
  __syncthreads();
  // cooperative weight gradient over the atoms of this block (same species), one coalesced
  // atomic per weight per block
  T* gw = grad + md.off_w[t];
  const T* S = reinterpret_cast<const T*>(smem_raw);
  for (int l = 0; l < Lq; l++) {
    const int in = md.in_of(t, l), out = md.width[l];
    const int woff = md.w_off(t, l), ho = md.h_off(l);
    const int hin_off = (l == 0) ? 0 : 3 * Fm + md.h_off(l - 1);            // x or h[l-1]
    const int hdin_off = (l == 0) ? Fm : 3 * Fm + Hs + md.h_off(l - 1);     // v or hd[l-1]
    const int dq_off = 3 * Fm + 3 * Hs + ho, dp_off = 3 * Fm + 4 * Hs + ho;
    for (int idx = threadIdx.x; idx < in * out + out; idx += ML_WARPS * 32) {
      T g = T(0);
      if (idx < in * out) {
        const int q = idx / out, j = idx - q * out;
#pragma unroll
        for (int a = 0; a < ML_WARPS; a++) {
          const T* A = S + (size_t)a * per;
          g += A[hin_off + q] * A[dq_off + j] + A[hdin_off + q] * A[dp_off + j];
        }
      } else {
        const int j = idx - in * out;
#pragma unroll
        for (int a = 0; a < ML_WARPS; a++) g += S[(size_t)a * per + dq_off + j];
      }
      atomicAdd(gw + woff + idx, g);
    }
  }
  for (int q = threadIdx.x; q < F; q += ML_WARPS * 32) {
    T g = T(0);
#pragma unroll
    for (int a = 0; a < ML_WARPS; a++) g -= S[(size_t)a * per + 2 * Fm + q];
    atomicAdd(grad + md.off_mu[t] + q, g);
  }
}

// ---------------------------------------------------------------------------- energy, loss
template <class T>
__device__ __forceinline__ T huber(T e) { T a = r_abs(e); return a <= T(1) ? T(0.5) * e * e : a - T(0.5); }
template <class T>
__device__ __forceinline__ T huber_d(T e) { return e > T(1) ? T(1) : (e < T(-1) ? T(-1) : e); }

// one block per frame: E_b = 0.5 * mean_i e_i (or 0.5 * sum), energy loss and its cotangent
template <class T>
__global__ void k_energy(int N, int nf, int per_atom, const T* __restrict__ e_atom, T* __restrict__ energy,
                         const T* __restrict__ e_label, T pe, int loss_kind, T* __restrict__ ebar,
                         double* __restrict__ losses, int* __restrict__ status) {
  __shared__ double red[9];
  const int b = blockIdx.x;
  double s = 0.0;
  for (int q = threadIdx.x; q < N; q += blockDim.x) s += (double)e_atom[(size_t)b * N + q];
  s = block_sum<double, 8>(s, red);
  if (threadIdx.x == 0) {
    const double Eb = per_atom ? 0.5 * s / N : 0.5 * s;
    if (!isfinite(Eb)) set_status(status, STAFB_ERR_NONFINITE);
    if (energy) energy[b] = (T)Eb;
    if (e_label) {
      const T e = (T)Eb - e_label[b];
      const T le = loss_kind == 0 ? huber(e) : e * e;
      const T de = loss_kind == 0 ? huber_d(e) : T(2) * e;
      atomicAdd(losses + 1, (double)le / nf);
      // cotangent on every atomic energy of the frame
      ebar[b] = pe * de / T(nf) * T(0.5) / (per_atom ? T(N) : T(1));
    }
  }
}

template <class T>
__global__ void k_force_loss(size_t n, const T* __restrict__ force, const T* __restrict__ f_label, T pf,
                             int loss_kind, T* __restrict__ fbar, double* __restrict__ losses) {
  __shared__ double red[9];
  double s = 0.0;
  const T scale = pf / T((double)n);
  for (size_t q = (size_t)blockIdx.x * blockDim.x + threadIdx.x; q < n; q += (size_t)gridDim.x * blockDim.x) {
    const T e = force[q] - f_label[q];
    s += (double)(loss_kind == 0 ? huber(e) : e * e);
    fbar[q] = scale * (loss_kind == 0 ? huber_d(e) : T(2) * e);
  }
  s = block_sum<double, 8>(s, red);
  if (threadIdx.x == 0) atomicAdd(losses + 3, s / (double)n);
}

// bound loss sum(alpha * [alpha > bound]) over alpha2b and alpha3b of every species
// (Keras ReLU(threshold): staf_models/staf_model.py:60-62,215-219) and its gradient
template <class T>
__global__ void k_bound(ModelDev md, const T* __restrict__ theta, T bound, T pb, T* __restrict__ grad,
                        double* __restrict__ losses) {
  __shared__ double red[9];
  double s = 0.0;
  for (int t = 0; t < md.nt; t++) {
    const int n2 = md.nt * md.Fr[t], n3 = md.C * 3 * md.Fa[t];
    for (int q = threadIdx.x; q < n2 + n3; q += blockDim.x) {
      const int idx = q < n2 ? md.off_a2[t] + q : md.off_a3[t] + (q - n2);
      const T x = theta[idx];
      if (x > bound) { s += (double)x; atomicAdd(grad + idx, pb); }
    }
  }
  s = block_sum<double, 8>(s, red);
  if (threadIdx.x == 0) losses[2] = s;
}

__global__ void k_finalize(double pe, double pf, double pb, double* __restrict__ losses) {
  losses[0] = pe * losses[1] + pb * losses[2] + pf * losses[3];
}

template <class T>
__global__ void k_adam(int n, T* __restrict__ theta, const T* __restrict__ grad, T* __restrict__ m,
                       T* __restrict__ v, T lr_t, T b1, T b2, T eps, T gscale) {
  const int q = blockIdx.x * blockDim.x + threadIdx.x;
  if (q >= n) return;
  const T g = grad[q] * gscale;
  const T mm = b1 * m[q] + (T(1) - b1) * g;
  const T vv = b2 * v[q] + (T(1) - b2) * g * g;
  m[q] = mm;
  v[q] = vv;
  theta[q] -= lr_t * mm / (r_sqrt(vv) + eps);
}

// Adam with the step count kept on the device, so that a captured CUDA graph can be replayed
template <class T>
__global__ void k_adam_dev(int n, T* __restrict__ theta, const T* __restrict__ grad, T* __restrict__ m,
                           T* __restrict__ v, double lr, double b1, double b2, T eps, T gscale,
                           const int* __restrict__ step_d) {
  const int q = blockIdx.x * blockDim.x + threadIdx.x;
  if (q >= n) return;
  const int step = *step_d + 1;
  const T lr_t = (T)(lr * sqrt(1.0 - pow(b2, (double)step)) / (1.0 - pow(b1, (double)step)));
  const T g = grad[q] * gscale;
  const T mm = (T)b1 * m[q] + (T(1) - (T)b1) * g;
  const T vv = (T)b2 * v[q] + (T(1) - (T)b2) * g * g;
  m[q] = mm;
  v[q] = vv;
  theta[q] -= lr_t * mm / (r_sqrt(vv) + eps);
}
__global__ void k_inc(int* p) { *p += 1; }

}  // namespace stafb

using namespace stafb;

struct stafb_model {
  stafb_ctx* ctx;
  ModelDev md;
  int n_params, n_emb;
  int blk_size[STAFB_MAX_TYPES];
  size_t es;
  // scratch for max_batch frames
  void *rad, *d3s, *af, *nd, *acts, *e_atom, *force, *fbar, *ebar, *gradnet, *gaf, *energy;
  int *im2, *ntr;
  double* losses_d;
  // staging for the *_host entry points
  void *pos_d, *box_d, *el_d, *fl_d;
  void* pin;  // pinned staging: pos | box | e_label | f_label
  double* losses_h;
  size_t smem_limit;
};

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
  const size_t es = m->es, A = (size_t)c->max_batch * d.N, nr = c->nr;
  STAFB_CUDA_OK(cudaMalloc(&m->rad, es * A * nr));
  STAFB_CUDA_OK(cudaMalloc(&m->d3s, es * A * nr));
  STAFB_CUDA_OK(cudaMalloc((void**)&m->im2, sizeof(int) * A * (nr + 1)));
  STAFB_CUDA_OK(cudaMalloc((void**)&m->ntr, sizeof(int) * A));
  STAFB_CUDA_OK(cudaMalloc(&m->af, es * A * d.Fmax));
  STAFB_CUDA_OK(cudaMalloc(&m->nd, es * A * d.Fmax));
  STAFB_CUDA_OK(cudaMalloc(&m->gradnet, es * A * d.Fmax));
  STAFB_CUDA_OK(cudaMalloc(&m->gaf, es * A * d.Fmax));
  STAFB_CUDA_OK(cudaMalloc(&m->acts, es * A * d.Hsum));
  STAFB_CUDA_OK(cudaMalloc(&m->e_atom, es * A));
  STAFB_CUDA_OK(cudaMalloc(&m->force, es * A * 3));
  STAFB_CUDA_OK(cudaMalloc(&m->fbar, es * A * 3));
  STAFB_CUDA_OK(cudaMalloc(&m->ebar, es * c->max_batch));
  STAFB_CUDA_OK(cudaMalloc(&m->energy, es * c->max_batch));
  STAFB_CUDA_OK(cudaMalloc((void**)&m->losses_d, sizeof(double) * 4));
  STAFB_CUDA_OK(cudaMalloc(&m->pos_d, es * A * 3));
  STAFB_CUDA_OK(cudaMalloc(&m->box_d, es * c->max_batch * 6));
  STAFB_CUDA_OK(cudaMalloc(&m->el_d, es * c->max_batch));
  STAFB_CUDA_OK(cudaMalloc(&m->fl_d, es * A * 3));
  STAFB_CUDA_OK(cudaMallocHost(&m->pin, es * (A * 6 + (size_t)c->max_batch * 7)));
  STAFB_CUDA_OK(cudaMallocHost((void**)&m->losses_h, sizeof(double) * 4));
  int dev = 0, lim = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&lim, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
  m->smem_limit = (size_t)lim;
  *out = m;
  return STAFB_OK;
}

extern "C" void stafb_model_destroy(stafb_model* m) {
  if (!m) return;
  void* ptrs[] = {m->rad, m->d3s, m->im2, m->ntr, m->af, m->nd, m->gradnet, m->gaf, m->acts, m->e_atom, m->force,
                  m->fbar, m->ebar, m->energy, m->losses_d, m->pos_d, m->box_d, m->el_d, m->fl_d};
  for (void* p : ptrs) cudaFree(p);
  cudaFreeHost(m->pin);
  cudaFreeHost(m->losses_h);
  free(m);
}

extern "C" int stafb_model_n_params(const stafb_model* m) { return m ? m->n_params : -1; }
extern "C" int stafb_model_n_emb(const stafb_model* m) { return m ? m->n_emb : -1; }
extern "C" void stafb_model_offsets(const stafb_model* m, int t, int out6[6]) {
  out6[0] = m->md.off_a2[t]; out6[1] = m->md.off_a3[t]; out6[2] = m->md.off_mu[t]; out6[3] = m->md.off_w[t];
  out6[4] = m->md.off_emb[t]; out6[5] = m->blk_size[t];
}

template <class T, int MODE>
static int launch_sweep(stafb_model* m, cudaStream_t s, int nf, const SweepIn<T>& in, const T* theta, const T* emb,
                        const T* chan_in, const T* fbar, T* out, T* grad) {
  const ModelDev& d = m->md;
  const int xt = MODE == MODE_FORCE ? 3 : (MODE == MODE_FGRAD ? 4 : 0);
  const int nacc = d.Famax + d.nt * d.Frmax + d.C * 3 * d.Famax;
  SweepLayout L = sweep_layout<T>(in.nr, d.nt, xt, nacc, d.Famax > 0 ? d.Famax : 1);
  const size_t sm = (size_t)L.total * SW_WARPS;
  if (sm > m->smem_limit) return STAFB_ERR_CAPACITY;
  static bool attr[2][4] = {{false}};
  if (sm > 48 * 1024 && !attr[sizeof(T) == 8][MODE]) {
    STAFB_CUDA_OK(cudaFuncSetAttribute(k_sweep<T, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       (int)m->smem_limit));
    attr[sizeof(T) == 8][MODE] = true;
  }
  const int blocks = species_blocks(d, nf, SW_WARPS);
  k_sweep<T, MODE><<<blocks, SW_WARPS * 32, sm, s>>>(d, in, L, theta, emb, chan_in, fbar, out, grad);
  m->ctx->launches++;
  return STAFB_OK;
}

template <class T>
static int run_fused(stafb_ctx* c, stafb_model* m, cudaStream_t s, const T* pos, const T* box, int nf,
                     const T* theta, const T* emb, int per_atom, bool train, const T* e_label, const T* f_label,
                     double pe, double pf, double pb, double bound, int loss_kind, double* losses_d, T* grad,
                     T* energy_out, T* force_out) {
  if (!c || !m || !pos || !box || !theta || !emb || nf <= 0) return STAFB_ERR_INVALID;
  if (nf > c->max_batch) return STAFB_ERR_CAPACITY;
  if (train && (!e_label || !f_label || !grad || !losses_d)) return STAFB_ERR_INVALID;
  const ModelDev& d = m->md;
  const int N = d.N;
  c->launches = 0;
  c->n_phase = 0;
  auto mark = [&]() {
    if (c->timing && c->n_phase < 16) cudaEventRecord(c->ev[c->n_phase++], s);
  };
  mark();
  T* rad = (T*)m->rad; T* d3s = (T*)m->d3s;
  int rc = launch_descriptors<T>(c, s, pos, box, nf, N, rad, nullptr, d3s, m->im2, nullptr, nullptr, nullptr,
                                 nullptr, m->ntr);
  if (rc != STAFB_OK) return rc;
  mark();  // descriptors
  SweepIn<T> in;
  in.geom = (const T*)c->geom; in.gsc = (const T*)c->gsc; in.rad = rad; in.d3s = d3s; in.im2 = m->im2; in.ntr = m->ntr;
  in.nf = nf; in.nr = c->nr;
  T* af = (T*)m->af; T* nd = (T*)m->nd; T* acts = (T*)m->acts; T* e_atom = (T*)m->e_atom;
  T* force = force_out ? force_out : (T*)m->force;
  T* energy = energy_out ? energy_out : (T*)m->energy;
  rc = launch_sweep<T, MODE_AF>(m, s, nf, in, theta, emb, nullptr, nullptr, af, nullptr);
  if (rc != STAFB_OK) return rc;
  mark();  // af_fwd
  const int mblocks = species_blocks(d, nf, ML_WARPS);
  {
    const size_t sm = sizeof(T) * (size_t)(d.Fmax + d.Hsum + 2 * d.maxw) * ML_WARPS;
    if (sm > m->smem_limit) return STAFB_ERR_CAPACITY;
    static bool attr[2] = {false, false};
    if (sm > 48 * 1024 && !attr[sizeof(T) == 8]) {
      STAFB_CUDA_OK(cudaFuncSetAttribute(k_mlp_fwd<T>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)m->smem_limit));
      attr[sizeof(T) == 8] = true;
    }
    k_mlp_fwd<T><<<mblocks, ML_WARPS * 32, sm, s>>>(d, nf, theta, af, acts, e_atom, nd);
    c->launches++;
  }
  mark();  // mlp_fwd
  STAFB_CUDA_OK(cudaMemsetAsync(force, 0, sizeof(T) * (size_t)nf * 3 * N, s));
  rc = launch_sweep<T, MODE_FORCE>(m, s, nf, in, theta, emb, nd, nullptr, force, nullptr);
  if (rc != STAFB_OK) return rc;
  mark();  // force
  if (train) {
    STAFB_CUDA_OK(cudaMemsetAsync(losses_d, 0, sizeof(double) * 4, s));
    STAFB_CUDA_OK(cudaMemsetAsync(grad, 0, sizeof(T) * (size_t)m->n_params, s));
  }
  k_energy<T><<<nf, 256, 0, s>>>(N, nf, per_atom, e_atom, energy, train ? e_label : nullptr, (T)pe, loss_kind,
                                 (T*)m->ebar, losses_d, c->status_d);
  c->launches++;
  if (train) {
    const size_t nF = (size_t)nf * 3 * N;
    int fb = (int)((nF + 255) / 256);
    if (fb > 1184) fb = 1184;
    k_force_loss<T><<<fb, 256, 0, s>>>(nF, force, f_label, (T)pf, loss_kind, (T*)m->fbar, losses_d);
    k_bound<T><<<1, 256, 0, s>>>(d, theta, (T)bound, (T)pb, grad, losses_d);
    c->launches += 2;
    mark();  // loss
    T* gradnet = (T*)m->gradnet;
    T* gaf = (T*)m->gaf;
    rc = launch_sweep<T, MODE_FGRAD>(m, s, nf, in, theta, emb, nd, (const T*)m->fbar, gradnet, grad);
    if (rc != STAFB_OK) return rc;
    mark();  // force_grad
    {
      const size_t sm = sizeof(T) * (size_t)(3 * d.Fmax + 5 * d.Hsum + 2 * d.maxw) * ML_WARPS;
      if (sm > m->smem_limit) return STAFB_ERR_CAPACITY;
      static bool attr[2] = {false, false};
      if (sm > 48 * 1024 && !attr[sizeof(T) == 8]) {
        STAFB_CUDA_OK(cudaFuncSetAttribute(k_mlp_bwd<T>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           (int)m->smem_limit));
        attr[sizeof(T) == 8] = true;
      }
      k_mlp_bwd<T><<<mblocks, ML_WARPS * 32, sm, s>>>(d, nf, theta, af, acts, (const T*)m->ebar, gradnet, gaf, grad);
      c->launches++;
    }
    mark();  // mlp_bwd
    rc = launch_sweep<T, MODE_AFGRAD>(m, s, nf, in, theta, emb, gaf, nullptr, nullptr, grad);
    if (rc != STAFB_OK) return rc;
    k_finalize<<<1, 1, 0, s>>>(pe, pf, pb, losses_d);
    c->launches++;
    mark();  // af_grad
  }
  STAFB_CUDA_OK(cudaGetLastError());
  return STAFB_OK;
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

extern "C" int stafb_train_step_host(stafb_ctx* c, stafb_model* m, void* stream, const void* pos_h,
                                     const void* box_h, int nf, const void* theta, const void* emb,
                                     const void* el_h, const void* fl_h, double pe, double pf, double pb,
                                     double bound, int loss_kind, double* losses_h, void* grad) {
  if (!c || !m || !pos_h || !box_h || !el_h || !fl_h || !losses_h) return STAFB_ERR_INVALID;
  if (nf > c->max_batch) return STAFB_ERR_CAPACITY;
  cudaStream_t s = (cudaStream_t)stream;
  const size_t es = m->es, A = (size_t)nf * m->md.N;
  // stage through pinned memory so that the copies are truly asynchronous
  char* pin = (char*)m->pin;
  char* p_pos = pin;
  char* p_fl = p_pos + es * A * 3;
  char* p_box = p_fl + es * A * 3;
  char* p_el = p_box + es * (size_t)nf * 6;
  memcpy(p_pos, pos_h, es * A * 3);
  memcpy(p_fl, fl_h, es * A * 3);
  memcpy(p_box, box_h, es * (size_t)nf * 6);
  memcpy(p_el, el_h, es * (size_t)nf);
  STAFB_CUDA_OK(cudaMemcpyAsync(m->pos_d, p_pos, es * A * 3, cudaMemcpyHostToDevice, s));
  STAFB_CUDA_OK(cudaMemcpyAsync(m->fl_d, p_fl, es * A * 3, cudaMemcpyHostToDevice, s));
  STAFB_CUDA_OK(cudaMemcpyAsync(m->box_d, p_box, es * (size_t)nf * 6, cudaMemcpyHostToDevice, s));
  STAFB_CUDA_OK(cudaMemcpyAsync(m->el_d, p_el, es * (size_t)nf, cudaMemcpyHostToDevice, s));
  int rc = stafb_train_step(c, m, stream, m->pos_d, m->box_d, nf, theta, emb, m->el_d, m->fl_d, pe, pf, pb, bound,
                            loss_kind, m->losses_d, grad, nullptr, nullptr);
  if (rc != STAFB_OK) return rc;
  STAFB_CUDA_OK(cudaMemcpyAsync(m->losses_h, m->losses_d, sizeof(double) * 4, cudaMemcpyDeviceToHost, s));
  STAFB_CUDA_OK(cudaMemcpyAsync(c->status_h, c->status_d, sizeof(int), cudaMemcpyDeviceToHost, s));
  STAFB_CUDA_OK(cudaStreamSynchronize(s));
  for (int q = 0; q < 4; q++) losses_h[q] = m->losses_h[q];
  if (*c->status_h != STAFB_OK) {
    int st = *c->status_h;
    cudaMemsetAsync(c->status_d, 0, sizeof(int), s);
    return st;
  }
  return STAFB_OK;
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
    k_adam_dev<float><<<(n + 255) / 256, 256, 0, s>>>(n, (float*)theta, (const float*)grad, (float*)mm, (float*)vv, lr,
                                                      b1, b2, (float)eps, (float)gscale, step_d);
  else
    k_adam_dev<double><<<(n + 255) / 256, 256, 0, s>>>(n, (double*)theta, (const double*)grad, (double*)mm,
                                                       (double*)vv, lr, b1, b2, eps, gscale, step_d);
  k_inc<<<1, 1, 0, s>>>(step_d);
  STAFB_CUDA_OK(cudaGetLastError());
  return STAFB_OK;
}
