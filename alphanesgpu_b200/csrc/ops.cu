// The reference's fingerprint / force / gradient operators on materialised descriptor tensors
// (the drop-in operator boundary).  Arithmetic follows
//   STAF/src/fingerprint/{rad,ang}/reforce.cu.cc, STAF/src/force/{rad,ang}/reforce.cu.cc,
//   STAF/src/grad_finger/{rad,ang}/reforce.cu.cc, STAF/src/grad_force/{rad,ang}/reforce.cu.cc
// of the reference; the execution plan does not: one warp (radial) or one block (angular)
// owns a central atom, reduces in registers / shared memory, and touches global memory with
// one write per output element (per-atom outputs) or one atomic per block (parameter
// gradients) instead of one global atomic per (neighbour, channel).  Channel/class pairs whose
// squared embedding is exactly zero are skipped (they contribute exactly zero).
#include "common.cuh"

namespace stafb {

constexpr int OPS_THREADS = 128;
constexpr int OPS_WARPS = OPS_THREADS / 32;

// Extra inputs / outputs of the ...Virial and ...VirialGrad operators (null pointers: plain operator).
template <class T>
struct VirArgs {
  const T* pos = nullptr;   // [nf,3N] Cartesian positions
  const T* box = nullptr;   // [nf,6]
  T* virial = nullptr;      // force ops: [nf,9] accumulated, W_ab -= g_a r_b
  const T* wbar = nullptr;  // grad ops: [nf,9] cotangent on the virial
};

// r_i - r_j with the minimum image taken in fractional space, as the reference's virial kernels form it
// (STAF/include/staf_force_pbc.cuh:15-49)
template <class T>
__device__ __forceinline__ void mic_cart(const T* __restrict__ pi, const T* __restrict__ pj, const T* __restrict__ B,
                                         T* d) {
  const T i0 = T(1.) / B[0], i1 = -B[1] / (B[0] * B[3]);
  const T i2 = (B[1] * B[4]) / (B[0] * B[3] * B[5]) - B[2] / (B[0] * B[5]);
  const T i3 = T(1.) / B[3], i4 = -B[4] / (B[3] * B[5]), i5 = T(1.) / B[5];
  T rx = (i0 * pi[0] + i1 * pi[1] + i2 * pi[2]) - (i0 * pj[0] + i1 * pj[1] + i2 * pj[2]);
  T ry = (i3 * pi[1] + i4 * pi[2]) - (i3 * pj[1] + i4 * pj[2]);
  T rz = i5 * pi[2] - i5 * pj[2];
  rx -= r_rint(rx); ry -= r_rint(ry); rz -= r_rint(rz);
  d[0] = B[0] * rx + B[1] * ry + B[2] * rz;
  d[1] = B[3] * ry + B[4] * rz;
  d[2] = B[5] * rz;
}

__device__ __forceinline__ int species_shift(const int* tipos, const int* actual_type) {
  int at = actual_type[0], s = 0;
  for (int y = 0; y < at; y++) s += tipos[y];
  return s;
}

// ---------------------------------------------------------------- radial AF (ComputeSortProj)
template <class T>
__global__ void __launch_bounds__(OPS_THREADS)
    k_af_rad(int natoms, int nr, int Fr, const T* __restrict__ rad, const int* __restrict__ im2,
             const T* __restrict__ alpha2b, const T* __restrict__ e2, const int* __restrict__ type_map,
             T* __restrict__ out) {
  const int gi = blockIdx.x * OPS_WARPS + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (gi >= natoms) return;
  const size_t base = gi;
  int n = im2[base * (nr + 1)];
  if (n > nr) n = nr;
  for (int c = 0; c < Fr; c++) {
    T acc = T(0);
    for (int j = lane; j < n; j += 32) {
      const T d = rad[base * nr + j];
      const int tj = type_map[im2[base * (nr + 1) + 1 + j]];
      const T ch = e2[Fr * tj + c];
      if (ch != T(0)) acc += d * (r_exp(alpha2b[Fr * tj + c] * d) * ch);
    }
    acc = warp_sum(acc);
    if (lane == 0) out[base * Fr + c] = acc;
  }
}

// Shared staging for the angular operators: species and cutoff value of the sorted
// neighbours, and the (j,k) pair of every triplet slot packed in 16 bits.
template <class T>
struct AngStage {
  int m, Tn;
  int* tj;             // [nr]
  T* ds;               // [nr]
  unsigned short* jk;  // [na]
};

template <class T>
__device__ __forceinline__ void ang_stage(AngStage<T>& st, size_t base, int nr, int na, const int* numtriplet,
                                          const int* im2, const T* ds3, const int* type_map) {
  int m = numtriplet[base];
  if (m > nr) m = nr;
  long long Tl = (long long)m * (m - 1) / 2;
  st.m = m;
  st.Tn = Tl < na ? (int)Tl : na;
  for (int k = threadIdx.x; k < m; k += blockDim.x) {
    st.tj[k] = type_map[im2[base * (nr + 1) + 1 + k]];
    st.ds[k] = ds3[base * nr + k];
  }
  for (int nn = threadIdx.x; nn < st.Tn; nn += blockDim.x) {
    int j, k;
    unrank_pair(nn, m, j, k);
    st.jk[nn] = (unsigned short)((j << 8) | k);
  }
  __syncthreads();
}

// ---------------------------------------------------------------- angular AF (ComputeSortProj3body)
template <class T>
__global__ void __launch_bounds__(OPS_THREADS)
    k_af_ang(int nr, int na, int Fa, int ncls, const T* __restrict__ ang, const T* __restrict__ ds3,
             const int* __restrict__ im2, const T* __restrict__ alpha3b, const T* __restrict__ e3,
             const int* __restrict__ type_map, const int* __restrict__ numtriplet, T* __restrict__ out) {
  extern __shared__ unsigned char smem_raw[];
  __shared__ T red[OPS_WARPS + 1];
  AngStage<T> st;
  st.ds = reinterpret_cast<T*>(smem_raw);
  st.tj = reinterpret_cast<int*>(st.ds + nr);
  st.jk = reinterpret_cast<unsigned short*>(st.tj + nr);
  const size_t base = blockIdx.x;
  ang_stage(st, base, nr, na, numtriplet, im2, ds3, type_map);
  const T* t_row = ang + base * na;
  for (int c = 0; c < Fa; c++) {
    T acc = T(0);
    for (int s = 0; s < ncls; s++) {
      const T ch = e3[s * Fa + c];
      if (ch == T(0)) continue;
      const T a1 = alpha3b[(s * Fa + c) * 3], a2 = alpha3b[(s * Fa + c) * 3 + 1], be = alpha3b[(s * Fa + c) * 3 + 2];
      for (int nn = threadIdx.x; nn < st.Tn; nn += OPS_THREADS) {
        const int j = st.jk[nn] >> 8, k = st.jk[nn] & 255;
        if (st.tj[j] + st.tj[k] != s) continue;
        const T t = t_row[nn], dj = st.ds[j], dk = st.ds[k];
        T sw = r_exp(a1 * dj + a2 * dk);
        sw += r_exp(a2 * dj + a1 * dk);
        sw *= r_exp(be * t);
        acc += t * sw * ch / T(2.);
      }
    }
    acc = block_sum<T, OPS_WARPS>(acc, red);
    if (threadIdx.x == 0) out[base * Fa + c] = acc;
  }
}

// ---------------------------------------------------------------- radial force (ComputeForceRadial)
template <class T>
__global__ void __launch_bounds__(OPS_THREADS)
    k_force_rad(int natoms, int Nl, int N, int nr, int Fr, const T* __restrict__ netderiv,
                const T* __restrict__ der2b, const int* __restrict__ im2, const T* __restrict__ rad,
                const T* __restrict__ alpha2b, const T* __restrict__ e2, const int* __restrict__ type_map,
                const int* __restrict__ tipos, const int* __restrict__ actual_type, T* __restrict__ force,
                VirArgs<T> va) {
  const int gi = blockIdx.x * OPS_WARPS + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (gi >= natoms) return;
  const int b = gi / Nl, par = gi - b * Nl;
  const int ipar = par + species_shift(tipos, actual_type);
  const size_t base = gi;
  int n = im2[base * (nr + 1)];
  if (n > nr) n = nr;
  T fx = T(0), fy = T(0), fz = T(0);
  T vw[9];
#pragma unroll
  for (int c = 0; c < 9; c++) vw[c] = T(0);
  for (int j = lane; j < n; j += 32) {
    const int nj = im2[base * (nr + 1) + 1 + j];
    const int tj = type_map[nj];
    const T d = rad[base * nr + j];
    T w = T(0);
    for (int c = 0; c < Fr; c++) {
      const T ch = e2[Fr * tj + c];
      if (ch == T(0)) continue;
      const T al = alpha2b[Fr * tj + c];
      T sds = ch * r_exp(al * d);
      sds *= (T(1.) + al * d);
      w += netderiv[base * Fr + c] * (T(0.5) * sds);
    }
    const T gx = w * der2b[(base * 3 + 0) * nr + j];
    const T gy = w * der2b[(base * 3 + 1) * nr + j];
    const T gz = w * der2b[(base * 3 + 2) * nr + j];
    T* fj = force + ((size_t)b * N + nj) * 3;
    atomicAdd(fj + 0, gx);
    atomicAdd(fj + 1, gy);
    atomicAdd(fj + 2, gz);
    fx -= gx; fy -= gy; fz -= gz;
    if (va.virial) {  // W_ab -= g_a r_b (force/rad/reforce.cu.cc:174-287)
      T r[3];
      mic_cart(va.pos + ((size_t)b * N + ipar) * 3, va.pos + ((size_t)b * N + nj) * 3, va.box + (size_t)b * 6, r);
      const T g[3] = {gx, gy, gz};
#pragma unroll
      for (int a = 0; a < 3; a++)
#pragma unroll
        for (int c = 0; c < 3; c++) vw[a * 3 + c] -= g[a] * r[c];
    }
  }
  fx = warp_sum(fx); fy = warp_sum(fy); fz = warp_sum(fz);
  if (lane == 0) {
    T* fi = force + ((size_t)b * N + ipar) * 3;
    atomicAdd(fi + 0, fx);
    atomicAdd(fi + 1, fy);
    atomicAdd(fi + 2, fz);
  }
  if (va.virial) {
#pragma unroll
    for (int c = 0; c < 9; c++) {
      const T v = warp_sum(vw[c]);
      if (lane == 0) atomicAdd(va.virial + (size_t)b * 9 + c, v);
    }
  }
}

// ---------------------------------------------------------------- angular force (ComputeForceTripl)
template <class T>
__global__ void __launch_bounds__(OPS_THREADS)
    k_force_ang(int Nl, int N, int nr, int na, int Fa, const T* __restrict__ netderiv, const T* __restrict__ ds3,
                const T* __restrict__ ang, const T* __restrict__ der3bsupp, const T* __restrict__ der3b,
                const int* __restrict__ im2, const T* __restrict__ alpha3b, const T* __restrict__ e3,
                const int* __restrict__ type_map, const int* __restrict__ tipos, const int* __restrict__ actual_type,
                const int* __restrict__ numtriplet, T* __restrict__ force, VirArgs<T> va) {
  extern __shared__ unsigned char smem_raw[];
  __shared__ T red[OPS_WARPS + 1];
  typedef typename Vec2<T>::type T2;
  AngStage<T> st;
  st.ds = reinterpret_cast<T*>(smem_raw);
  T* dsup = st.ds + nr;       // [3][nr] der3bsupp row
  T* fnb = dsup + 3 * nr;     // [nr][3] neighbour force accumulators
  T* nd = fnb + 3 * nr;       // [Fa]
  st.tj = reinterpret_cast<int*>(nd + Fa);
  int* ids = st.tj + nr;
  st.jk = reinterpret_cast<unsigned short*>(ids + nr);
  const size_t base = blockIdx.x;
  const int b = (int)(base / Nl), par = (int)(base - (size_t)b * Nl);
  const int ipar = par + species_shift(tipos, actual_type);
  for (int k = threadIdx.x; k < nr; k += OPS_THREADS) {
    ids[k] = im2[base * (nr + 1) + 1 + k];
    for (int a = 0; a < 3; a++) {
      dsup[a * nr + k] = der3bsupp[(base * 3 + a) * nr + k];
      fnb[k * 3 + a] = T(0);
    }
  }
  for (int c = threadIdx.x; c < Fa; c += OPS_THREADS) nd[c] = netderiv[base * Fa + c];
  ang_stage(st, base, nr, na, numtriplet, im2, ds3, type_map);
  const T2* d3 = reinterpret_cast<const T2*>(der3b) + base * 3 * na;
  T fx = T(0), fy = T(0), fz = T(0);
  for (int nn = threadIdx.x; nn < st.Tn; nn += OPS_THREADS) {
    const int j = st.jk[nn] >> 8, k = st.jk[nn] & 255;
    const int s = st.tj[j] + st.tj[k];
    const T t = ang[base * na + nn], rj = st.ds[j], rk = st.ds[k];
    T D = T(0), BJ = T(0), BK = T(0);
    for (int c = 0; c < Fa; c++) {
      const T ch = e3[s * Fa + c];
      if (ch == T(0)) continue;
      const T ax = alpha3b[(s * Fa + c) * 3], ay = alpha3b[(s * Fa + c) * 3 + 1], az = alpha3b[(s * Fa + c) * 3 + 2];
      const T w = T(0.5) * nd[c] * ch;
      const T eb = r_exp(az * t);
      const T sim1 = r_exp(ay * rj + ax * rk), sim2 = r_exp(ax * rj + ay * rk);
      D += w * (eb * (T(1.) + az * t) * (sim1 + sim2) * T(0.5));
      BJ += w * ((ax * sim2 + ay * sim1) * eb * T(0.5) * t);
      BK += w * ((ax * sim1 + ay * sim2) * eb * T(0.5) * t);
    }
    T fj[3], fk[3];
#pragma unroll
    for (int a = 0; a < 3; a++) {
      const T2 id = d3[(size_t)a * na + nn];
      fj[a] = D * id.x + BJ * dsup[a * nr + j];
      fk[a] = D * id.y + BK * dsup[a * nr + k];
      atomicAdd(&fnb[j * 3 + a], fj[a]);
      atomicAdd(&fnb[k * 3 + a], fk[a]);
    }
    fx -= fj[0] + fk[0];
    fy -= fj[1] + fk[1];
    fz -= fj[2] + fk[2];
  }
  fx = block_sum<T, OPS_WARPS>(fx, red);
  fy = block_sum<T, OPS_WARPS>(fy, red);
  fz = block_sum<T, OPS_WARPS>(fz, red);
  __syncthreads();
  T* fb = force + (size_t)b * N * 3;
  for (int q = threadIdx.x; q < st.m * 3; q += OPS_THREADS) atomicAdd(fb + (size_t)ids[q / 3] * 3 + (q % 3), fnb[q]);
  if (threadIdx.x == 0) {
    atomicAdd(fb + (size_t)ipar * 3 + 0, fx);
    atomicAdd(fb + (size_t)ipar * 3 + 1, fy);
    atomicAdd(fb + (size_t)ipar * 3 + 2, fz);
  }
  if (va.virial && threadIdx.x < 32) {
    // W_ab -= f_ij,a r_ij,b + f_ik,a r_ik,b (force/ang/reforce.cu.cc:269-457): every force this centre puts on
    // neighbour k multiplies the same r_ik, so the per-neighbour totals suffice
    T w[9];
#pragma unroll
    for (int c = 0; c < 9; c++) w[c] = T(0);
    for (int k = threadIdx.x; k < st.m; k += 32) {
      T r[3];
      mic_cart(va.pos + ((size_t)b * N + ipar) * 3, va.pos + ((size_t)b * N + ids[k]) * 3, va.box + (size_t)b * 6, r);
#pragma unroll
      for (int a = 0; a < 3; a++)
#pragma unroll
        for (int c = 0; c < 3; c++) w[a * 3 + c] -= fnb[k * 3 + a] * r[c];
    }
#pragma unroll
    for (int c = 0; c < 9; c++) {
      const T v = warp_sum(w[c]);
      if (threadIdx.x == 0) atomicAdd(va.virial + (size_t)b * 9 + c, v);
    }
  }
}

// ---------------------------------------------------------------- d/d(alpha2b) of the radial AF (ComputeTwoBodyParGrad)
template <class T>
__global__ void __launch_bounds__(OPS_THREADS)
    k_grad_af_rad(int natoms, int nr, int Fr, int nt, const T* __restrict__ prevgrad, const T* __restrict__ rad,
                  const int* __restrict__ im2, const T* __restrict__ alpha2b, const T* __restrict__ e2,
                  const int* __restrict__ type_map, T* __restrict__ g_alpha, T* __restrict__ g_emb) {
  const int gi = blockIdx.x * OPS_WARPS + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (gi >= natoms) return;
  const size_t base = gi;
  int n = im2[base * (nr + 1)];
  if (n > nr) n = nr;
  for (int c = 0; c < Fr; c++) {
    const T pg = prevgrad[base * Fr + c];
    T ga[STAFB_MAX_TYPES], ge[STAFB_MAX_TYPES];
#pragma unroll
    for (int t = 0; t < STAFB_MAX_TYPES; t++) ga[t] = ge[t] = T(0);
    for (int j = lane; j < n; j += 32) {
      const T d = rad[base * nr + j];
      const int tj = type_map[im2[base * (nr + 1) + 1 + j]];
      const T ex = r_exp(alpha2b[tj * Fr + c] * d);
      const T va = d * d * (ex * e2[tj * Fr + c] * pg);
      const T ve = d * (ex * pg);
#pragma unroll
      for (int t = 0; t < STAFB_MAX_TYPES; t++)
        if (t == tj) { ga[t] += va; ge[t] += ve; }
    }
#pragma unroll
    for (int t = 0; t < STAFB_MAX_TYPES; t++) {
      if (t >= nt) break;
      const T sa = warp_sum(ga[t]), se = warp_sum(ge[t]);
      if (lane == 0) {
        if (sa != T(0)) atomicAdd(g_alpha + t * Fr + c, sa);
        if (se != T(0)) atomicAdd(g_emb + t * Fr + c, se);
      }
    }
  }
}

// ---------------------------------------------------------------- d/d(alpha3b) of the angular AF (ComputeSortProj3bodyGrad)
template <class T>
__global__ void __launch_bounds__(OPS_THREADS)
    k_grad_af_ang(int nr, int na, int Fa, int ncls, const T* __restrict__ prevgrad, const T* __restrict__ ang,
                  const T* __restrict__ ds3, const int* __restrict__ im2, const T* __restrict__ alpha3b,
                  const T* __restrict__ e3, const int* __restrict__ type_map, const int* __restrict__ numtriplet,
                  T* __restrict__ g_alpha3) {
  extern __shared__ unsigned char smem_raw[];
  __shared__ T red[OPS_WARPS + 1];
  AngStage<T> st;
  st.ds = reinterpret_cast<T*>(smem_raw);
  st.tj = reinterpret_cast<int*>(st.ds + nr);
  st.jk = reinterpret_cast<unsigned short*>(st.tj + nr);
  const size_t base = blockIdx.x;
  ang_stage(st, base, nr, na, numtriplet, im2, ds3, type_map);
  const T* t_row = ang + base * na;
  for (int c = 0; c < Fa; c++) {
    const T pg = prevgrad[base * Fa + c];
    for (int s = 0; s < ncls; s++) {
      const T ch = e3[s * Fa + c];
      if (ch == T(0)) continue;
      const T a1 = alpha3b[(s * Fa + c) * 3], a2 = alpha3b[(s * Fa + c) * 3 + 1], be = alpha3b[(s * Fa + c) * 3 + 2];
      T g1 = T(0), g2 = T(0), g3 = T(0);
      for (int nn = threadIdx.x; nn < st.Tn; nn += OPS_THREADS) {
        const int j = st.jk[nn] >> 8, k = st.jk[nn] & 255;
        if (st.tj[j] + st.tj[k] != s) continue;
        const T t = t_row[nn], dj = st.ds[j], dy = st.ds[k];
        const T e12 = r_exp(a1 * dj + a2 * dy), e21 = r_exp(a1 * dy + a2 * dj), bt = r_exp(be * t);
        const T common = pg * ch * bt * t / T(2.);
        g1 += common * (e12 * dj + e21 * dy);
        g2 += common * (e12 * dy + e21 * dj);
        g3 += common * (e12 + e21) * t;
      }
      g1 = block_sum<T, OPS_WARPS>(g1, red);
      g2 = block_sum<T, OPS_WARPS>(g2, red);
      g3 = block_sum<T, OPS_WARPS>(g3, red);
      if (threadIdx.x == 0) {
        atomicAdd(g_alpha3 + (s * Fa + c) * 3 + 0, g1);
        atomicAdd(g_alpha3 + (s * Fa + c) * 3 + 1, g2);
        atomicAdd(g_alpha3 + (s * Fa + c) * 3 + 2, g3);
      }
    }
  }
}

// ---------------------------------------------------------------- backward of the radial force (ComputeForceRadialGrad)
template <class T>
__global__ void __launch_bounds__(OPS_THREADS)
    k_grad_force_rad(int natoms, int Nl, int N, int nr, int Fr, int nt, const T* __restrict__ prevgrad,
                     const T* __restrict__ netderiv, const T* __restrict__ der2b, const int* __restrict__ im2,
                     const T* __restrict__ rad, const T* __restrict__ alpha2b, const T* __restrict__ e2,
                     const int* __restrict__ type_map, const int* __restrict__ tipos,
                     const int* __restrict__ actual_type, T* __restrict__ gradnet, T* __restrict__ g_alpha,
                     T* __restrict__ g_emb, VirArgs<T> va) {
  const int gi = blockIdx.x * OPS_WARPS + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (gi >= natoms) return;
  const int b = gi / Nl, par = gi - b * Nl;
  const int ipar = par + species_shift(tipos, actual_type);
  const size_t base = gi;
  int n = im2[base * (nr + 1)];
  if (n > nr) n = nr;
  const T* pgb = prevgrad + (size_t)b * N * 3;
  const T pix = pgb[ipar * 3], piy = pgb[ipar * 3 + 1], piz = pgb[ipar * 3 + 2];
  // q_j = sum_a (Fbar_j - Fbar_i)_a * 0.5 * dd/dr_{i,a}, per neighbour (two slots per lane cover nr <= 64;
  // the loop handles any nr)
  for (int c = 0; c < Fr; c++) {
    const T NG = netderiv[base * Fr + c];
    T gn = T(0);
    T ga[STAFB_MAX_TYPES], ge[STAFB_MAX_TYPES];
#pragma unroll
    for (int t = 0; t < STAFB_MAX_TYPES; t++) ga[t] = ge[t] = T(0);
    for (int j = lane; j < n; j += 32) {
      const int nj = im2[base * (nr + 1) + 1 + j];
      const int tj = type_map[nj];
      const T d = rad[base * nr + j];
      T wd[3] = {T(0), T(0), T(0)};
      if (va.wbar) {  // the virial cotangent shifts the neighbour's force cotangent by -(Wbar r) (grad_force/rad/reforce.cu.cc:165-234)
        T r[3];
        mic_cart(va.pos + ((size_t)b * N + ipar) * 3, va.pos + ((size_t)b * N + nj) * 3, va.box + (size_t)b * 6, r);
        const T* Wg = va.wbar + (size_t)b * 9;
#pragma unroll
        for (int a = 0; a < 3; a++) wd[a] = Wg[a * 3] * r[0] + Wg[a * 3 + 1] * r[1] + Wg[a * 3 + 2] * r[2];
      }
      const T q = T(0.5) * ((pgb[nj * 3] - pix - wd[0]) * der2b[(base * 3 + 0) * nr + j] +
                            (pgb[nj * 3 + 1] - piy - wd[1]) * der2b[(base * 3 + 1) * nr + j] +
                            (pgb[nj * 3 + 2] - piz - wd[2]) * der2b[(base * 3 + 2) * nr + j]);
      const T al = alpha2b[Fr * tj + c], ch = e2[Fr * tj + c];
      const T s1 = r_exp(al * d);
      const T sds = s1 * (T(1.) + al * d);
      const T ba = ch * s1 * d * (T(2.) + al * d);
      gn += q * ch * sds;
      const T va = q * NG * ba, ve = q * NG * sds;
#pragma unroll
      for (int t = 0; t < STAFB_MAX_TYPES; t++)
        if (t == tj) { ga[t] += va; ge[t] += ve; }
    }
    gn = warp_sum(gn);
    if (lane == 0) gradnet[base * Fr + c] = gn;
#pragma unroll
    for (int t = 0; t < STAFB_MAX_TYPES; t++) {
      if (t >= nt) break;
      const T sa = warp_sum(ga[t]), se = warp_sum(ge[t]);
      if (lane == 0) {
        if (sa != T(0)) atomicAdd(g_alpha + t * Fr + c, sa);
        if (se != T(0)) atomicAdd(g_emb + t * Fr + c, se);
      }
    }
  }
}

// ---------------------------------------------------------------- backward of the angular force (ComputeForceTriplGrad)
// Per triplet the force cotangent enters only through three scalars,
//   Q  = sum_a (Fb_j-Fb_i)_a dt/d(ij)_a + (Fb_k-Fb_i)_a dt/d(ik)_a,
//   Pj = sum_a (Fb_j-Fb_i)_a dfc_j,a,   Pk = sum_a (Fb_k-Fb_i)_a dfc_k,a,
// staged once in shared memory; every (class, channel) sweep then costs three exponentials.
template <class T>
__global__ void __launch_bounds__(OPS_THREADS)
    k_grad_force_ang(int Nl, int N, int nr, int na, int Fa, int ncls, const T* __restrict__ prevgrad,
                     const T* __restrict__ netderiv, const T* __restrict__ ds3, const T* __restrict__ ang,
                     const T* __restrict__ der3bsupp, const T* __restrict__ der3b, const int* __restrict__ im2,
                     const T* __restrict__ alpha3b, const T* __restrict__ e3, const int* __restrict__ type_map,
                     const int* __restrict__ tipos, const int* __restrict__ actual_type,
                     const int* __restrict__ numtriplet, T* __restrict__ gradnet, T* __restrict__ g_alpha3,
                     VirArgs<T> va) {
  extern __shared__ unsigned char smem_raw[];
  __shared__ T red[OPS_WARPS + 1];
  typedef typename Vec2<T>::type T2;
  AngStage<T> st;
  st.ds = reinterpret_cast<T*>(smem_raw);
  T* pn = st.ds + nr;        // [nr] Pj per neighbour
  T* dF = pn + nr;           // [nr][3] Fbar_j - Fbar_i
  T* Q = dF + 3 * nr;        // [na]
  st.tj = reinterpret_cast<int*>(Q + na);
  st.jk = reinterpret_cast<unsigned short*>(st.tj + nr);
  const size_t base = blockIdx.x;
  const int b = (int)(base / Nl), par = (int)(base - (size_t)b * Nl);
  const int ipar = par + species_shift(tipos, actual_type);
  const T* pgb = prevgrad + (size_t)b * N * 3;
  for (int k = threadIdx.x; k < nr; k += OPS_THREADS) {
    const int id = im2[base * (nr + 1) + 1 + k];
    T p = T(0);
    T wd[3] = {T(0), T(0), T(0)};
    if (va.wbar && k < numtriplet[base]) {  // grad_force/ang/reforce.cu.cc:274-446
      T r[3];
      mic_cart(va.pos + ((size_t)b * N + ipar) * 3, va.pos + ((size_t)b * N + id) * 3, va.box + (size_t)b * 6, r);
      const T* Wg = va.wbar + (size_t)b * 9;
#pragma unroll
      for (int a = 0; a < 3; a++) wd[a] = Wg[a * 3] * r[0] + Wg[a * 3 + 1] * r[1] + Wg[a * 3 + 2] * r[2];
    }
    for (int a = 0; a < 3; a++) {
      const T d = pgb[id * 3 + a] - pgb[ipar * 3 + a] - wd[a];
      dF[k * 3 + a] = d;
      p += d * der3bsupp[(base * 3 + a) * nr + k];
    }
    pn[k] = p;
  }
  ang_stage(st, base, nr, na, numtriplet, im2, ds3, type_map);
  const T2* d3 = reinterpret_cast<const T2*>(der3b) + base * 3 * na;
  for (int nn = threadIdx.x; nn < st.Tn; nn += OPS_THREADS) {
    const int j = st.jk[nn] >> 8, k = st.jk[nn] & 255;
    T q = T(0);
#pragma unroll
    for (int a = 0; a < 3; a++) {
      const T2 id = d3[(size_t)a * na + nn];
      q += dF[j * 3 + a] * id.x + dF[k * 3 + a] * id.y;
    }
    Q[nn] = q;
  }
  __syncthreads();
  const T* t_row = ang + base * na;
  for (int c = 0; c < Fa; c++) {
    const T NG = netderiv[base * Fa + c];
    T gn = T(0);
    for (int s = 0; s < ncls; s++) {
      const T ch = e3[s * Fa + c];
      if (ch == T(0)) continue;
      const T ax = alpha3b[(s * Fa + c) * 3], ay = alpha3b[(s * Fa + c) * 3 + 1], az = alpha3b[(s * Fa + c) * 3 + 2];
      T g1 = T(0), g2 = T(0), g3 = T(0);
      for (int nn = threadIdx.x; nn < st.Tn; nn += OPS_THREADS) {
        const int j = st.jk[nn] >> 8, k = st.jk[nn] & 255;
        if (st.tj[j] + st.tj[k] != s) continue;
        const T t = t_row[nn], rj = st.ds[j], rk = st.ds[k];
        const T q = Q[nn], pj = pn[j], pk = pn[k];
        const T eb = r_exp(az * t);
        const T sim1 = r_exp(ay * rj + ax * rk), sim2 = r_exp(ax * rj + ay * rk);
        const T ss = sim1 + sim2;
        const T h = T(0.5) * ch;
        const T opb = T(1.) + az * t;
        const T delta = eb * opb * ss * T(0.5);
        const T suppj = (ax * sim2 + ay * sim1) * eb, suppk = (ax * sim1 + ay * sim2) * eb;
        const T Bj = suppj * t * T(0.5), Bk = suppk * t * T(0.5);
        gn += h * (delta * q + Bj * pj + Bk * pk);
        const T ba1 = eb * opb * (sim1 * rk + sim2 * rj) * T(0.5);
        const T ba2 = eb * opb * (sim1 * rj + sim2 * rk) * T(0.5);
        const T bb = eb * t * (T(2.) + az * t) * ss * T(0.5);
        const T et = eb * T(0.5) * t;
        const T a1j = (sim2 + ax * sim2 * rj + ay * sim1 * rk) * et;
        const T a2j = (sim1 + ay * sim1 * rj + ax * sim2 * rk) * et;
        const T a1k = (sim1 + ax * sim1 * rk + ay * sim2 * rj) * et;
        const T a2k = (sim2 + ay * sim2 * rk + ax * sim1 * rj) * et;
        const T hn = h * NG;
        g1 += hn * (ba1 * q + a1j * pj + a1k * pk);
        g2 += hn * (ba2 * q + a2j * pj + a2k * pk);
        g3 += hn * (bb * q + Bj * t * pj + Bk * t * pk);
      }
      g1 = block_sum<T, OPS_WARPS>(g1, red);
      g2 = block_sum<T, OPS_WARPS>(g2, red);
      g3 = block_sum<T, OPS_WARPS>(g3, red);
      if (threadIdx.x == 0) {
        atomicAdd(g_alpha3 + (s * Fa + c) * 3 + 0, g1);
        atomicAdd(g_alpha3 + (s * Fa + c) * 3 + 1, g2);
        atomicAdd(g_alpha3 + (s * Fa + c) * 3 + 2, g3);
      }
    }
    gn = block_sum<T, OPS_WARPS>(gn, red);
    if (threadIdx.x == 0) gradnet[base * Fa + c] = gn;
  }
}

// ================================================================= launchers
template <class T>
static int ops_check(stafb_ctx* c) {
  if (!c) return STAFB_ERR_INVALID;
  if ((c->dtype == STAFB_F32) != (sizeof(T) == 4)) return STAFB_ERR_INVALID;
  return STAFB_OK;
}

static inline int ncls_of(int nt) {
  int C = nt * (nt + 1) / 2, smax = 2 * nt - 1;
  return C < smax ? C : smax;
}

template <class T>
int op_sort_proj(stafb_ctx* c, cudaStream_t s, const T* rad, const int* im2, const T* a2, const T* e2,
                 const int* tm, int nf, int Nl, int nt, int Fr, T* out) {
  const int n = nf * Nl;
  if (n <= 0) return STAFB_OK;
  k_af_rad<T><<<(n + OPS_WARPS - 1) / OPS_WARPS, OPS_THREADS, 0, s>>>(n, c->nr, Fr, rad, im2, a2, e2, tm, out);
  STAFB_CUDA_OK(cudaGetLastError());
  return STAFB_OK;
}

template <class T>
int op_sort_proj3(stafb_ctx* c, cudaStream_t s, const T* ang, const T* ds3, const int* im2, const T* a3, const T* e3,
                  const int* tm, const int* ntr, int nf, int Nl, int nt, int Fa, T* out) {
  const int n = nf * Nl;
  if (n <= 0) return STAFB_OK;
  size_t sm = (size_t)c->nr * (sizeof(T) + sizeof(int)) + (size_t)c->na * 2;
  k_af_ang<T><<<n, OPS_THREADS, sm, s>>>(c->nr, c->na, Fa, ncls_of(nt), ang, ds3, im2, a3, e3, tm, ntr, out);
  STAFB_CUDA_OK(cudaGetLastError());
  return STAFB_OK;
}

template <class T>
int op_force_rad(stafb_ctx* c, cudaStream_t s, const T* nd, const T* der2b, const int* im2, const T* rad,
                 const T* a2, const T* e2, const int* tm, const int* tipos, const int* at, int nf, int Nl, int N,
                 int nt, int Fr, T* force, VirArgs<T> va = VirArgs<T>()) {
  STAFB_CUDA_OK(cudaMemsetAsync(force, 0, sizeof(T) * (size_t)nf * 3 * N, s));
  if (va.virial) STAFB_CUDA_OK(cudaMemsetAsync(va.virial, 0, sizeof(T) * (size_t)nf * 9, s));
  const int n = nf * Nl;
  if (n <= 0) return STAFB_OK;
  k_force_rad<T><<<(n + OPS_WARPS - 1) / OPS_WARPS, OPS_THREADS, 0, s>>>(n, Nl, N, c->nr, Fr, nd, der2b, im2, rad, a2,
                                                                        e2, tm, tipos, at, force, va);
  STAFB_CUDA_OK(cudaGetLastError());
  return STAFB_OK;
}

template <class T>
int op_force_ang(stafb_ctx* c, cudaStream_t s, const T* nd, const T* ds3, const T* ang, const T* d3s, const T* d3,
                 const int* im2, const T* a3, const T* e3, const int* tm, const int* tipos, const int* at,
                 const int* ntr, int nf, int Nl, int N, int nt, int Fa, T* force, VirArgs<T> va = VirArgs<T>()) {
  STAFB_CUDA_OK(cudaMemsetAsync(force, 0, sizeof(T) * (size_t)nf * 3 * N, s));
  if (va.virial) STAFB_CUDA_OK(cudaMemsetAsync(va.virial, 0, sizeof(T) * (size_t)nf * 9, s));
  const int n = nf * Nl;
  if (n <= 0) return STAFB_OK;
  size_t sm = sizeof(T) * ((size_t)c->nr * 7 + Fa) + sizeof(int) * (size_t)c->nr * 2 + (size_t)c->na * 2;
  k_force_ang<T><<<n, OPS_THREADS, sm, s>>>(Nl, N, c->nr, c->na, Fa, nd, ds3, ang, d3s, d3, im2, a3, e3, tm, tipos, at,
                                            ntr, force, va);
  STAFB_CUDA_OK(cudaGetLastError());
  return STAFB_OK;
}

template <class T>
int op_grad_af_rad(stafb_ctx* c, cudaStream_t s, const T* pg, const T* rad, const int* im2, const T* a2, const T* e2,
                   const int* tm, int nf, int Nl, int nt, int Fr, T* ga, T* ge) {
  if (nt > STAFB_MAX_TYPES) return STAFB_ERR_INVALID;
  STAFB_CUDA_OK(cudaMemsetAsync(ga, 0, sizeof(T) * nt * Fr, s));
  STAFB_CUDA_OK(cudaMemsetAsync(ge, 0, sizeof(T) * nt * Fr, s));
  const int n = nf * Nl;
  if (n <= 0) return STAFB_OK;
  k_grad_af_rad<T><<<(n + OPS_WARPS - 1) / OPS_WARPS, OPS_THREADS, 0, s>>>(n, c->nr, Fr, nt, pg, rad, im2, a2, e2, tm,
                                                                          ga, ge);
  STAFB_CUDA_OK(cudaGetLastError());
  return STAFB_OK;
}

template <class T>
int op_grad_af_ang(stafb_ctx* c, cudaStream_t s, const T* pg, const T* ang, const T* ds3, const int* im2,
                   const T* a3, const T* e3, const int* tm, const int* ntr, int nf, int Nl, int nt, int Fa, T* ga,
                   T* ge) {
  const int C = nt * (nt + 1) / 2;
  STAFB_CUDA_OK(cudaMemsetAsync(ga, 0, sizeof(T) * C * 3 * Fa, s));
  STAFB_CUDA_OK(cudaMemsetAsync(ge, 0, sizeof(T) * C * Fa, s));
  const int n = nf * Nl;
  if (n <= 0) return STAFB_OK;
  size_t sm = (size_t)c->nr * (sizeof(T) + sizeof(int)) + (size_t)c->na * 2;
  k_grad_af_ang<T><<<n, OPS_THREADS, sm, s>>>(c->nr, c->na, Fa, ncls_of(nt), pg, ang, ds3, im2, a3, e3, tm, ntr, ga);
  STAFB_CUDA_OK(cudaGetLastError());
  return STAFB_OK;
}

template <class T>
int op_grad_force_rad(stafb_ctx* c, cudaStream_t s, const T* pg, const T* nd, const T* der2b, const int* im2,
                      const T* rad, const T* a2, const T* e2, const int* tm, const int* tipos, const int* at, int nf,
                      int Nl, int N, int nt, int Fr, T* gradnet, T* ga, T* ge, VirArgs<T> va = VirArgs<T>()) {
  if (nt > STAFB_MAX_TYPES) return STAFB_ERR_INVALID;
  STAFB_CUDA_OK(cudaMemsetAsync(ga, 0, sizeof(T) * nt * Fr, s));
  STAFB_CUDA_OK(cudaMemsetAsync(ge, 0, sizeof(T) * nt * Fr, s));
  const int n = nf * Nl;
  if (n <= 0) return STAFB_OK;
  k_grad_force_rad<T><<<(n + OPS_WARPS - 1) / OPS_WARPS, OPS_THREADS, 0, s>>>(n, Nl, N, c->nr, Fr, nt, pg, nd, der2b,
                                                                             im2, rad, a2, e2, tm, tipos, at, gradnet,
                                                                             ga, ge, va);
  STAFB_CUDA_OK(cudaGetLastError());
  return STAFB_OK;
}

template <class T>
int op_grad_force_ang(stafb_ctx* c, cudaStream_t s, const T* pg, const T* nd, const T* ds3, const T* ang,
                      const T* d3s, const T* d3, const int* im2, const T* a3, const T* e3, const int* tm,
                      const int* tipos, const int* at, const int* ntr, int nf, int Nl, int N, int nt, int Fa,
                      T* gradnet, T* ga, T* gck, VirArgs<T> va = VirArgs<T>()) {
  const int C = nt * (nt + 1) / 2;
  STAFB_CUDA_OK(cudaMemsetAsync(ga, 0, sizeof(T) * C * 3 * Fa, s));
  STAFB_CUDA_OK(cudaMemsetAsync(gck, 0, sizeof(T) * C * Fa, s));
  const int n = nf * Nl;
  if (n <= 0) return STAFB_OK;
  size_t sm = sizeof(T) * ((size_t)c->nr * 5 + c->na) + sizeof(int) * (size_t)c->nr + (size_t)c->na * 2;
  static bool attr_done[64] = {false};  // per instantiation and device: the attribute belongs to the current device
  int dev = 0;
  cudaGetDevice(&dev);
  bool& done = attr_done[(dev >= 0 && dev < 64) ? dev : 0];
  if (sm > 48 * 1024 && !done) {
    STAFB_CUDA_OK(cudaFuncSetAttribute(k_grad_force_ang<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    done = true;
  }
  k_grad_force_ang<T><<<n, OPS_THREADS, sm, s>>>(Nl, N, c->nr, c->na, Fa, ncls_of(nt), pg, nd, ds3, ang, d3s, d3, im2,
                                                 a3, e3, tm, tipos, at, ntr, gradnet, ga, va);
  STAFB_CUDA_OK(cudaGetLastError());
  return STAFB_OK;
}

}  // namespace stafb

using namespace stafb;
#define DISPATCH(c, call_f, call_d)                               \
  do {                                                            \
    if (!(c)) return STAFB_ERR_INVALID;                           \
    cudaStream_t s = (cudaStream_t)stream;                        \
    if ((c)->dtype == STAFB_F32) { typedef float R; return call_f; } \
    typedef double R;                                             \
    return call_d;                                                \
  } while (0)

extern "C" int stafb_compute_sort_proj(stafb_ctx* c, void* stream, const void* rad, const int* im2, const void* a2,
                                       const void* e2, const int* tm, int nf, int Nl, int nt, int Fr, void* out) {
  DISPATCH(c, op_sort_proj<R>(c, s, (const R*)rad, im2, (const R*)a2, (const R*)e2, tm, nf, Nl, nt, Fr, (R*)out),
           op_sort_proj<R>(c, s, (const R*)rad, im2, (const R*)a2, (const R*)e2, tm, nf, Nl, nt, Fr, (R*)out));
}

extern "C" int stafb_compute_sort_proj3body(stafb_ctx* c, void* stream, const void* ang, const void* ds3,
                                            const int* im3, const int* im2, const void* a3, const void* e3,
                                            const int* tm, const int* ntr, int nf, int Nl, int nt, int Fa,
                                            void* out) {
  (void)im3;  // the pair ids are recomputed from interaction_map_rad; same values by construction
  DISPATCH(c,
           op_sort_proj3<R>(c, s, (const R*)ang, (const R*)ds3, im2, (const R*)a3, (const R*)e3, tm, ntr, nf, Nl, nt,
                            Fa, (R*)out),
           op_sort_proj3<R>(c, s, (const R*)ang, (const R*)ds3, im2, (const R*)a3, (const R*)e3, tm, ntr, nf, Nl, nt,
                            Fa, (R*)out));
}

extern "C" int stafb_compute_force_radial(stafb_ctx* c, void* stream, const void* nd, const void* der2b,
                                          const int* im2, const void* rad, const void* a2, const void* e2,
                                          const int* tm, const int* tipos, const int* at, int nf, int Nl, int N,
                                          int nt, int Fr, void* force) {
  DISPATCH(c,
           op_force_rad<R>(c, s, (const R*)nd, (const R*)der2b, im2, (const R*)rad, (const R*)a2, (const R*)e2, tm,
                           tipos, at, nf, Nl, N, nt, Fr, (R*)force),
           op_force_rad<R>(c, s, (const R*)nd, (const R*)der2b, im2, (const R*)rad, (const R*)a2, (const R*)e2, tm,
                           tipos, at, nf, Nl, N, nt, Fr, (R*)force));
}

extern "C" int stafb_compute_force_tripl(stafb_ctx* c, void* stream, const void* nd, const void* ds3, const void* ang,
                                         const void* d3s, const void* d3, const int* im2, const int* im3,
                                         const void* a3, const void* e3, const int* tm, const int* tipos,
                                         const int* at, const int* ntr, int nf, int Nl, int N, int nt, int Fa,
                                         void* force) {
  (void)im3;
  DISPATCH(c,
           op_force_ang<R>(c, s, (const R*)nd, (const R*)ds3, (const R*)ang, (const R*)d3s, (const R*)d3, im2,
                           (const R*)a3, (const R*)e3, tm, tipos, at, ntr, nf, Nl, N, nt, Fa, (R*)force),
           op_force_ang<R>(c, s, (const R*)nd, (const R*)ds3, (const R*)ang, (const R*)d3s, (const R*)d3, im2,
                           (const R*)a3, (const R*)e3, tm, tipos, at, ntr, nf, Nl, N, nt, Fa, (R*)force));
}

extern "C" int stafb_compute_two_body_par_grad(stafb_ctx* c, void* stream, const void* pg, const void* rad,
                                               const int* im2, const void* a2, const void* e2, const int* tm, int nf,
                                               int Nl, int nt, int Fr, void* ga, void* ge) {
  DISPATCH(c,
           op_grad_af_rad<R>(c, s, (const R*)pg, (const R*)rad, im2, (const R*)a2, (const R*)e2, tm, nf, Nl, nt, Fr,
                             (R*)ga, (R*)ge),
           op_grad_af_rad<R>(c, s, (const R*)pg, (const R*)rad, im2, (const R*)a2, (const R*)e2, tm, nf, Nl, nt, Fr,
                             (R*)ga, (R*)ge));
}

extern "C" int stafb_compute_sort_proj3body_grad(stafb_ctx* c, void* stream, const void* pg, const void* ang,
                                                 const void* ds3, const int* im3, const int* im2, const void* a3,
                                                 const void* e3, const int* tm, const int* ntr, int nf, int Nl,
                                                 int nt, int Fa, void* ga, void* ge) {
  (void)im3;
  DISPATCH(c,
           op_grad_af_ang<R>(c, s, (const R*)pg, (const R*)ang, (const R*)ds3, im2, (const R*)a3, (const R*)e3, tm,
                             ntr, nf, Nl, nt, Fa, (R*)ga, (R*)ge),
           op_grad_af_ang<R>(c, s, (const R*)pg, (const R*)ang, (const R*)ds3, im2, (const R*)a3, (const R*)e3, tm,
                             ntr, nf, Nl, nt, Fa, (R*)ga, (R*)ge));
}

extern "C" int stafb_compute_force_radial_grad(stafb_ctx* c, void* stream, const void* pg, const void* nd,
                                               const void* der2b, const int* im2, const void* rad, const void* a2,
                                               const void* e2, const int* tm, const int* tipos, const int* at,
                                               int nf, int Nl, int N, int nt, int Fr, void* gradnet, void* ga,
                                               void* ge) {
  DISPATCH(c,
           op_grad_force_rad<R>(c, s, (const R*)pg, (const R*)nd, (const R*)der2b, im2, (const R*)rad, (const R*)a2,
                                (const R*)e2, tm, tipos, at, nf, Nl, N, nt, Fr, (R*)gradnet, (R*)ga, (R*)ge),
           op_grad_force_rad<R>(c, s, (const R*)pg, (const R*)nd, (const R*)der2b, im2, (const R*)rad, (const R*)a2,
                                (const R*)e2, tm, tipos, at, nf, Nl, N, nt, Fr, (R*)gradnet, (R*)ga, (R*)ge));
}

extern "C" int stafb_compute_force_tripl_grad(stafb_ctx* c, void* stream, const void* pg, const void* nd,
                                              const void* ds3, const void* ang, const void* d3s, const void* d3,
                                              const int* im2, const int* im3, const void* a3, const void* e3,
                                              const int* tm, const int* tipos, const int* at, const int* ntr, int nf,
                                              int Nl, int N, int nt, int Fa, void* gradnet, void* ga, void* gck) {
  (void)im3;
  DISPATCH(c,
           op_grad_force_ang<R>(c, s, (const R*)pg, (const R*)nd, (const R*)ds3, (const R*)ang, (const R*)d3s,
                                (const R*)d3, im2, (const R*)a3, (const R*)e3, tm, tipos, at, ntr, nf, Nl, N, nt, Fa,
                                (R*)gradnet, (R*)ga, (R*)gck),
           op_grad_force_ang<R>(c, s, (const R*)pg, (const R*)nd, (const R*)ds3, (const R*)ang, (const R*)d3s,
                                (const R*)d3, im2, (const R*)a3, (const R*)e3, tm, tipos, at, ntr, nf, Nl, N, nt, Fa,
                                (R*)gradnet, (R*)ga, (R*)gck));
}


// ---- ...Virial / ...VirialGrad variants: the same kernels with the positions, the box and the virial (or its
// cotangent) attached
template <class R>
static VirArgs<R> vir_args(const void* pos, const void* box, void* virial, const void* wbar) {
  VirArgs<R> va;
  va.pos = (const R*)pos; va.box = (const R*)box; va.virial = (R*)virial; va.wbar = (const R*)wbar;
  return va;
}

extern "C" int stafb_compute_force_radial_virial(stafb_ctx* c, void* stream, const void* nd, const void* der2b,
                                                 const int* im2, const void* rad, const void* a2, const void* e2,
                                                 const int* tm, const int* tipos, const int* at, const void* pos,
                                                 const void* box, int nf, int Nl, int N, int nt, int Fr, void* force,
                                                 void* virial) {
  if (!pos || !box || !virial) return STAFB_ERR_INVALID;
  DISPATCH(c,
           op_force_rad<R>(c, s, (const R*)nd, (const R*)der2b, im2, (const R*)rad, (const R*)a2, (const R*)e2, tm,
                           tipos, at, nf, Nl, N, nt, Fr, (R*)force, vir_args<R>(pos, box, virial, nullptr)),
           op_force_rad<R>(c, s, (const R*)nd, (const R*)der2b, im2, (const R*)rad, (const R*)a2, (const R*)e2, tm,
                           tipos, at, nf, Nl, N, nt, Fr, (R*)force, vir_args<R>(pos, box, virial, nullptr)));
}

extern "C" int stafb_compute_force_tripl_virial(stafb_ctx* c, void* stream, const void* nd, const void* ds3,
                                                const void* ang, const void* d3s, const void* d3, const int* im2,
                                                const int* im3, const void* a3, const void* e3, const int* tm,
                                                const int* tipos, const int* at, const int* ntr, const void* pos,
                                                const void* box, int nf, int Nl, int N, int nt, int Fa, void* force,
                                                void* virial) {
  (void)im3;
  if (!pos || !box || !virial) return STAFB_ERR_INVALID;
  DISPATCH(c,
           op_force_ang<R>(c, s, (const R*)nd, (const R*)ds3, (const R*)ang, (const R*)d3s, (const R*)d3, im2,
                           (const R*)a3, (const R*)e3, tm, tipos, at, ntr, nf, Nl, N, nt, Fa, (R*)force,
                           vir_args<R>(pos, box, virial, nullptr)),
           op_force_ang<R>(c, s, (const R*)nd, (const R*)ds3, (const R*)ang, (const R*)d3s, (const R*)d3, im2,
                           (const R*)a3, (const R*)e3, tm, tipos, at, ntr, nf, Nl, N, nt, Fa, (R*)force,
                           vir_args<R>(pos, box, virial, nullptr)));
}

extern "C" int stafb_compute_force_radial_virial_grad(stafb_ctx* c, void* stream, const void* pg, const void* pgv,
                                                      const void* nd, const void* der2b, const int* im2,
                                                      const void* rad, const void* a2, const void* e2, const int* tm,
                                                      const int* tipos, const int* at, const void* pos,
                                                      const void* box, int nf, int Nl, int N, int nt, int Fr,
                                                      void* gradnet, void* ga, void* ge) {
  if (!pos || !box || !pgv) return STAFB_ERR_INVALID;
  DISPATCH(c,
           op_grad_force_rad<R>(c, s, (const R*)pg, (const R*)nd, (const R*)der2b, im2, (const R*)rad, (const R*)a2,
                                (const R*)e2, tm, tipos, at, nf, Nl, N, nt, Fr, (R*)gradnet, (R*)ga, (R*)ge,
                                vir_args<R>(pos, box, nullptr, pgv)),
           op_grad_force_rad<R>(c, s, (const R*)pg, (const R*)nd, (const R*)der2b, im2, (const R*)rad, (const R*)a2,
                                (const R*)e2, tm, tipos, at, nf, Nl, N, nt, Fr, (R*)gradnet, (R*)ga, (R*)ge,
                                vir_args<R>(pos, box, nullptr, pgv)));
}

extern "C" int stafb_compute_force_tripl_virial_grad(stafb_ctx* c, void* stream, const void* pg, const void* pgv,
                                                     const void* nd, const void* ds3, const void* ang,
                                                     const void* d3s, const void* d3, const int* im2, const int* im3,
                                                     const void* a3, const void* e3, const int* tm, const int* tipos,
                                                     const int* at, const int* ntr, const void* pos, const void* box,
                                                     int nf, int Nl, int N, int nt, int Fa, void* gradnet, void* ga,
                                                     void* gck) {
  (void)im3;
  if (!pos || !box || !pgv) return STAFB_ERR_INVALID;
  DISPATCH(c,
           op_grad_force_ang<R>(c, s, (const R*)pg, (const R*)nd, (const R*)ds3, (const R*)ang, (const R*)d3s,
                                (const R*)d3, im2, (const R*)a3, (const R*)e3, tm, tipos, at, ntr, nf, Nl, N, nt, Fa,
                                (R*)gradnet, (R*)ga, (R*)gck, vir_args<R>(pos, box, nullptr, pgv)),
           op_grad_force_ang<R>(c, s, (const R*)pg, (const R*)nd, (const R*)ds3, (const R*)ang, (const R*)d3s,
                                (const R*)d3, im2, (const R*)a3, (const R*)e3, tm, tipos, at, ntr, nf, Nl, N, nt, Fa,
                                (R*)gradnet, (R*)ga, (R*)gck, vir_args<R>(pos, box, nullptr, pgv)));
}
