// Neighbour list + radial / angular descriptors (op ComputeDescriptorsLight).
//
// Follows the arithmetic of STAF/src/descriptor_builder/celle_gpu.cu.cc:11-260 and
// STAF/src/descriptor_builder/reforce.cu.cc:17-236 of the reference, with a different
// execution plan: no host synchronisation (the inverse box and the cell grid are computed on
// the device), all frames in one launch, one warp per central atom that discovers, sorts and
// describes its own neighbour row in shared memory, and a CSR cell list whose slot order is
// made deterministic (ascending atom index) so that ties in dist2 resolve reproducibly.
//
// This translation unit is compiled with -fmad=false: positions, squared distances and the
// cutoff tests must round in expression order, because neighbour sets and neighbour ORDER
// are compared bit-exactly.
#include <string.h>
#include "common.cuh"

namespace stafb {

template <class T>
__device__ void frame_geometry(const T* __restrict__ B, int N, T cutoff, int cell_cap, FrameGeom<T>& g, int* status) {
  for (int q = 0; q < 6; q++) g.box[q] = B[q];
  if (!(B[0] != T(0) && B[3] != T(0) && B[5] != T(0))) {
    set_status(status, STAFB_ERR_BAD_BOX);
    for (int q = 0; q < 6; q++) g.inv[q] = T(0);
    g.nx = g.ny = g.nz = 3;
    g.ncell = 27;
    g.sx = g.sy = g.sz = T(1) / T(3);
    return;
  }
  // inverse of the upper-triangular box: descriptor_builder/reforce.cc:283-299
  g.inv[0] = T(1.) / B[0];
  g.inv[1] = -B[1] / (B[0] * B[3]);
  g.inv[2] = (B[1] * B[4]) / (B[0] * B[3] * B[5]) - B[2] / (B[0] * B[5]);
  g.inv[3] = T(1.) / B[3];
  g.inv[4] = -B[4] / (B[3] * B[5]);
  g.inv[5] = T(1.) / B[5];
  // cell counts: celle_gpu.cu.cc:208-228
  T volume = B[0] * B[3] * B[5];
  int cx = (int)(volume / (r_sqrt(B[3] * B[3] * B[5] * B[5] + B[5] * B[5] * B[1] * B[1] +
                                  B[3] * B[3] * B[2] * B[2] + B[4] * B[4] * B[1] * B[1]) *
                           cutoff));
  int cy = (int)(volume / (B[0] * r_sqrt(B[5] * B[5] + B[4] * B[4]) * cutoff));
  int cz = (int)(volume / (B[0] * B[3] * cutoff));
  while ((cx * cy * cz > 27) && (cx * cy * cz > N)) {
    if (cx > cy) {
      if (cx > cz) cx--; else cz--;
    } else {
      if (cy > cz) cy--; else cz--;
    }
  }
  if (cx < 3) cx = 3;
  if (cy < 3) cy = 3;
  if (cz < 3) cz = 3;
  if ((long long)cx * cy * cz > cell_cap) {
    set_status(status, STAFB_ERR_CAPACITY);
    cx = cy = cz = 3;
  }
  g.nx = cx; g.ny = cy; g.nz = cz;
  g.ncell = cx * cy * cz;
  g.sx = T(1.) / (T)cx;
  g.sy = T(1.) / (T)cy;
  g.sz = T(1.) / (T)cz;
}

// Frame geometry, fractional coordinates (celle_gpu.cu.cc:11-28) and the cell of every atom
// (celle_gpu.cu.cc:176-201) in one launch: grid (blocks over atoms, frames); every block derives its
// frame's geometry again (a few dozen flops) instead of waiting for a separate set-up launch.
template <class T>
__global__ void k_cells(const T* __restrict__ pos, const T* __restrict__ box, int nf, int N, T cutoff, int cell_cap,
                        FrameGeom<T>* __restrict__ fg, T* __restrict__ frac, int* __restrict__ cell_of,
                        int* __restrict__ cell_count, int* __restrict__ status) {
  __shared__ FrameGeom<T> gs;
  const int b = blockIdx.y;
  chain_wait();
  if (threadIdx.x == 0) {
    frame_geometry<T>(box + 6 * b, N, cutoff, cell_cap, gs, status);
    if (blockIdx.x == 0) fg[b] = gs;
  }
  __syncthreads();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= N) return;
  const FrameGeom<T>& g = gs;
  const size_t t = (size_t)b * N + i;
  T px = pos[t * 3 + 0], py = pos[t * 3 + 1], pz = pos[t * 3 + 2];
  T fx = (g.inv[0] * px + g.inv[1] * py + g.inv[2] * pz);
  T fy = (g.inv[3] * py + g.inv[4] * pz);
  T fz = (g.inv[5] * pz);
  frac[t * 3 + 0] = fx;
  frac[t * 3 + 1] = fy;
  frac[t * 3 + 2] = fz;
  int cx = (int)r_floor(fx / g.sx);
  cx = cx % g.nx;
  if (cx < 0) cx += g.nx;
  int cy = (int)r_floor(fy / g.sy);
  cy = cy % g.ny;
  if (cy < 0) cy += g.ny;
  int cz = (int)r_floor(fz / g.sz);
  cz = cz % g.nz;
  if (cz < 0) cz += g.nz;
  int c = cx + cy * g.nx + cz * (g.nx * g.ny);
  cell_of[t] = c;
  atomicAdd(cell_count + (size_t)b * cell_cap + c, 1);
}

// Members of every cell in ascending atom index, gathered directly by one warp per cell that walks
// the frame's atoms 32 at a time (used for small systems; replaces the fill + sort pair).
template <class T>
__global__ void k_gather_cells(const FrameGeom<T>* __restrict__ fg, int nf, int N, const int* __restrict__ cell_of,
                               const int* __restrict__ cell_start, int* __restrict__ cells_sorted, int cell_cap) {
  chain_wait();
  int gw = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  int b = gw / cell_cap, c = gw - b * cell_cap;
  if (b >= nf || c >= fg[b].ncell) return;
  const int* co = cell_of + (size_t)b * N;
  int* dst = cells_sorted + (size_t)b * N + cell_start[(size_t)b * (cell_cap + 1) + c];
  const unsigned lt = (1u << lane) - 1u;
  int cnt = 0;
  for (int j0 = 0; j0 < N; j0 += 32) {
    const int j = j0 + lane;
    const bool p = (j < N) && (co[j] == c);
    const unsigned bal = __ballot_sync(0xffffffffu, p);
    if (p) dst[cnt + __popc(bal & lt)] = j;
    cnt += __popc(bal);
  }
}

// Small systems: frame geometry, fractional coordinates, cell of every atom, per-cell counts, their
// exclusive scan and the members of every cell in ascending atom index - one block per frame, all
// bookkeeping in shared memory (k_cells + k_scan + k_gather_cells in one launch, no counter memset).
// Dynamic shared memory: (cell_cap + 1 + N) ints.
template <class T>
__global__ void __launch_bounds__(1024)
    k_cell_lists_small(const T* __restrict__ pos, const T* __restrict__ box, int N, T cutoff, int cell_cap, int mpc,
                       FrameGeom<T>* __restrict__ fg, T* __restrict__ frac, int* __restrict__ cell_of,
                       int* __restrict__ cell_start, int* __restrict__ cells_sorted, int* __restrict__ status) {
  extern __shared__ int sm_i[];
  __shared__ FrameGeom<T> gs;
  __shared__ int part[32];
  __shared__ int carry;
  int* cnt = sm_i;                  // [cell_cap + 1] counts, then exclusive starts
  int* cof = sm_i + cell_cap + 1;   // [N] cell of every atom
  const int b = blockIdx.x, tid = threadIdx.x, lane = tid & 31, w = tid >> 5, nw = blockDim.x >> 5;
  if (tid == 0) {
    frame_geometry<T>(box + 6 * b, N, cutoff, cell_cap, gs, status);
    fg[b] = gs;
    carry = 0;
  }
  for (int c = tid; c <= cell_cap; c += blockDim.x) cnt[c] = 0;
  __syncthreads();
  const FrameGeom<T>& g = gs;
  for (int i = tid; i < N; i += blockDim.x) {
    const size_t t = (size_t)b * N + i;
    T px = pos[t * 3 + 0], py = pos[t * 3 + 1], pz = pos[t * 3 + 2];
    T fx = (g.inv[0] * px + g.inv[1] * py + g.inv[2] * pz);
    T fy = (g.inv[3] * py + g.inv[4] * pz);
    T fz = (g.inv[5] * pz);
    frac[t * 3 + 0] = fx;
    frac[t * 3 + 1] = fy;
    frac[t * 3 + 2] = fz;
    int cx = (int)r_floor(fx / g.sx);
    cx = cx % g.nx;
    if (cx < 0) cx += g.nx;
    int cy = (int)r_floor(fy / g.sy);
    cy = cy % g.ny;
    if (cy < 0) cy += g.ny;
    int cz = (int)r_floor(fz / g.sz);
    cz = cz % g.nz;
    if (cz < 0) cz += g.nz;
    const int c = cx + cy * g.nx + cz * (g.nx * g.ny);
    cell_of[t] = c;
    cof[i] = c;
    atomicAdd(&cnt[c], 1);
  }
  __syncthreads();
  const int ncell = g.ncell;
  int* st = cell_start + (size_t)b * (cell_cap + 1);
  for (int base = 0; base < ncell; base += blockDim.x) {
    const int c = base + tid;
    const int v = (c < ncell) ? cnt[c] : 0;
    if (v > mpc) set_status(status, STAFB_ERR_CELL_OVERFLOW);
    int x = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int y = __shfl_up_sync(0xffffffffu, x, o);
      if (lane >= o) x += y;
    }
    if (lane == 31) part[w] = x;
    __syncthreads();
    int off = carry;
    for (int q = 0; q < w; q++) off += part[q];
    if (c < ncell) {
      cnt[c] = off + x - v;
      st[c] = off + x - v;
    }
    __syncthreads();
    if (tid == 0) {
      int tot = 0;
      for (int q = 0; q < nw; q++) tot += part[q];
      carry += tot;
    }
    __syncthreads();
  }
  if (tid == 0) st[ncell] = carry;
  // members in ascending atom index: one warp per cell walks the frame's atoms 32 at a time
  const unsigned lt = (1u << lane) - 1u;
  int* dstb = cells_sorted + (size_t)b * N;
  for (int c = w; c < ncell; c += nw) {
    int* dst = dstb + cnt[c];
    int k = 0;
    for (int j0 = 0; j0 < N; j0 += 32) {
      const int j = j0 + lane;
      const bool p = (j < N) && (cof[j] == c);
      const unsigned bal = __ballot_sync(0xffffffffu, p);
      if (p) dst[k + __popc(bal & lt)] = j;
      k += __popc(bal);
    }
  }
}

// Exclusive scan of the per-cell counts of one frame (one block per frame).
template <class T>
__global__ void k_scan(const FrameGeom<T>* __restrict__ fg, const int* __restrict__ cell_count,
                       int* __restrict__ cell_start, int* __restrict__ cell_cursor, int cell_cap, int mpc,
                       int* __restrict__ status) {
  __shared__ int part[32];
  __shared__ int carry;
  chain_wait();
  const int b = blockIdx.x, ncell = fg[b].ncell;
  const int* cnt = cell_count + (size_t)b * cell_cap;
  int* st = cell_start + (size_t)b * (cell_cap + 1);
  int* cur = cell_cursor + (size_t)b * cell_cap;
  if (threadIdx.x == 0) carry = 0;
  __syncthreads();
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = blockDim.x >> 5;
  for (int base = 0; base < ncell; base += blockDim.x) {
    int c = base + threadIdx.x;
    int v = (c < ncell) ? cnt[c] : 0;
    if (v > mpc) set_status(status, STAFB_ERR_CELL_OVERFLOW);
    int x = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      int y = __shfl_up_sync(0xffffffffu, x, o);
      if (lane >= o) x += y;
    }
    if (lane == 31) part[w] = x;
    __syncthreads();
    int off = carry;
    for (int q = 0; q < w; q++) off += part[q];
    if (c < ncell) {
      st[c] = off + x - v;
      cur[c] = 0;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      int tot = 0;
      for (int q = 0; q < nw; q++) tot += part[q];
      carry += tot;
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) st[ncell] = carry;
}

__global__ void k_fill(int nf, int N, const int* __restrict__ cell_of, const int* __restrict__ cell_start,
                       int* __restrict__ cell_cursor, int* __restrict__ cells_raw, int cell_cap) {
  chain_wait();
  int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= nf * N) return;
  int b = t / N, i = t - b * N;
  int c = cell_of[t];
  int slot = atomicAdd(cell_cursor + (size_t)b * cell_cap + c, 1);
  cells_raw[(size_t)b * N + cell_start[(size_t)b * (cell_cap + 1) + c] + slot] = i;
}

// Orders every cell's members by atom index (one warp per cell): the reference's slot order
// is the atomicAdd arrival order (celle_gpu.cu.cc:197-200), restated as ascending index.
template <class T>
__global__ void k_sort_cells(const FrameGeom<T>* __restrict__ fg, int nf, int N, const int* __restrict__ cell_start,
                             const int* __restrict__ cells_raw, int* __restrict__ cells_sorted, int cell_cap) {
  chain_wait();
  int gw = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  int b = gw / cell_cap, c = gw - b * cell_cap;
  if (b >= nf || c >= fg[b].ncell) return;
  const int* st = cell_start + (size_t)b * (cell_cap + 1);
  int s0 = st[c], s1 = st[c + 1];
  const int* src = cells_raw + (size_t)b * N;
  int* dst = cells_sorted + (size_t)b * N;
  for (int e = s0 + lane; e < s1; e += 32) {
    int me = src[e], r = 0;
    for (int f = s0; f < s1; f++) r += (src[f] < me);
    dst[s0 + r] = me;
  }
}

template <class T>
__device__ __forceinline__ void mic_vec(const FrameGeom<T>& g, T ax, T ay, T az, T bx, T by, T bz, T& dx, T& dy,
                                        T& dz) {
  // a - b in fractional space, nearest image, back to Cartesian (celle_gpu.cu.cc:96-109)
  T ox = ax - bx, oy = ay - by, oz = az - bz;
  ox -= r_rint(ox);
  oy -= r_rint(oy);
  oz -= r_rint(oz);
  dx = g.box[0] * ox + g.box[1] * oy + g.box[2] * oz;
  dy = g.box[3] * oy + g.box[4] * oz;
  dz = g.box[5] * oz;
}

// What a fused sweep needs of one neighbour slot (the U and V entries of the record, common.cuh).
template <class T>
struct SlotVals {
  T ux, uy, uz, fc, rinv, dfc, d, dd;
};

// One slot of a central atom's radial row (reforce.cu.cc:17-110) from the vector v = r_i - r_j: radial
// descriptor, angular-support cutoff, their gradients, the neighbour id and the compact geometry the
// angular-descriptor kernel reads.  Slots past the neighbour count (valid == false) are zero-filled.  Every
// output pointer may be null; `sv` always receives the slot's values for the record of the fused sweeps.
template <class T>
__device__ __forceinline__ void radial_slot(const CoreCoef<T>& cc, bool valid, int j, T vx, T vy, T vz, size_t base,
                                            int k, int nr, T* __restrict__ raddescr, T* __restrict__ des3bsupp,
                                            int* __restrict__ intmap2b, T* __restrict__ der2b,
                                            T* __restrict__ der3bsupp, T* __restrict__ geom, T* __restrict__ gsc,
                                            int& nang, SlotVals<T>& sv) {
  const T PI = PIc<T>();
  T rd = T(0), d3 = T(0), g2x = T(0), g2y = T(0), g2z = T(0), g3x = T(0), g3y = T(0), g3z = T(0);
  T dn = T(0), s2 = T(0), s3 = T(0);
  if (valid) {
    dn = r_sqrt(vx * vx + vy * vy + vz * vz);
    if (dn < cc.Ra) {
      nang++;
      d3 = T(0.5) * (r_cos(PI * dn / cc.Ra) + T(1));
      const T pre = T(-0.5) * r_sin(PI * dn / cc.Ra) * PI / cc.Ra;
      s3 = pre;
      g3x = pre * vx / dn;
      g3y = pre * vy / dn;
      g3z = pre * vz / dn;
    }
    if (dn < cc.Rs) {
      // A/r^1 + B/r^-30 + C with the powers by repeated multiplication (the reference calls pow;
      // the exponents are the constants 1 and -30 of descriptor_builder/reforce.cc:102-103)
      const T r2 = dn * dn, r4 = r2 * r2, r8 = r4 * r4, r16 = r8 * r8;
      const T r28 = r16 * r8 * r4, r29 = r28 * dn, r30 = r28 * r2;
      rd = cc.A / dn + cc.B * r30 + cc.C;
      const T pre = (-cc.pa * cc.A / r2 - cc.pb * cc.B * r29);
      s2 = pre;
      g2x = pre * vx / dn;
      g2y = pre * vy / dn;
      g2z = pre * vz / dn;
    } else {
      rd = T(0.5) * (r_cos(PI * dn / cc.Rc) + T(1));
      const T pre = T(-0.5) * r_sin(PI * dn / cc.Rc) * PI / cc.Rc;
      s2 = pre;
      g2x = pre * vx / dn;
      g2y = pre * vy / dn;
      g2z = pre * vz / dn;
    }
  }
  if (raddescr) raddescr[base * nr + k] = rd;
  if (des3bsupp) des3bsupp[base * nr + k] = d3;
  if (der2b) {
    der2b[(base * 3 + 0) * nr + k] = g2x;
    der2b[(base * 3 + 1) * nr + k] = g2y;
    der2b[(base * 3 + 2) * nr + k] = g2z;
  }
  if (der3bsupp) {
    der3bsupp[(base * 3 + 0) * nr + k] = g3x;
    der3bsupp[(base * 3 + 1) * nr + k] = g3y;
    der3bsupp[(base * 3 + 2) * nr + k] = g3z;
  }
  if (intmap2b) intmap2b[base * (nr + 1) + 1 + k] = valid ? j : 0;
  if (geom) {
    typename Vec4<T>::type q;
    q.x = vx; q.y = vy; q.z = vz; q.w = dn;
    reinterpret_cast<typename Vec4<T>::type*>(geom)[base * nr + k] = q;
  }
  if (gsc) {
    // scalar radial derivatives: der2b = s2 * v/|v|, der3bsupp = s3 * v/|v|
    typename Vec2<T>::type q;
    q.x = s2; q.y = s3;
    reinterpret_cast<typename Vec2<T>::type*>(gsc)[base * nr + k] = q;
  }
  const T inv = valid ? T(1) / dn : T(0);
  sv.ux = vx * inv; sv.uy = vy * inv; sv.uz = vz * inv; sv.fc = d3;
  sv.rinv = inv; sv.dfc = s3; sv.d = rd; sv.dd = s2;
}

__device__ __forceinline__ int sink_species(const RowSink& sk, int j) {
  if (sk.tmap) return sk.tmap[j];
  int t = 0;
  while (t < sk.nt - 1 && j >= sk.shift[t + 1]) t++;
  return t;
}

// Positions of a distance-sorted row in the species-grouped order of the record: slot k of species q goes to
// (number of neighbours of species < q) + (number of species-q slots before k).  One warp; spos[k] receives
// position | species << 16 for k < n, cnt[q] the neighbours per species.  ids[k] = neighbour of sorted slot k.
__device__ __forceinline__ void group_by_species(const RowSink& sk, const int* ids, int n, int lane, int* spos,
                                                 int (&cnt)[STAFB_MAX_TYPES]) {
  const unsigned lt = (1u << lane) - 1u;
#pragma unroll
  for (int q = 0; q < STAFB_MAX_TYPES; q++) cnt[q] = 0;
  for (int k0 = 0; k0 < n; k0 += 32) {
    const int k = k0 + lane;
    const int sp = (k < n) ? sink_species(sk, ids[k]) : -1;
    int mine = 0;
#pragma unroll
    for (int q = 0; q < STAFB_MAX_TYPES; q++) {
      const unsigned bal = __ballot_sync(0xffffffffu, sp == q);
      if (sp == q) mine = cnt[q] + __popc(bal & lt);
      cnt[q] += __popc(bal);
    }
    if (k < n) spos[k] = mine | (sp << 16);  // rank inside the species for now
  }
  __syncwarp();
  int off[STAFB_MAX_TYPES];
  off[0] = 0;
#pragma unroll
  for (int q = 1; q < STAFB_MAX_TYPES; q++) off[q] = off[q - 1] + cnt[q - 1];
  for (int k = lane; k < n; k += 32) {
    const int v = spos[k], sp = v >> 16;
    int o = 0;
#pragma unroll
    for (int q = 0; q < STAFB_MAX_TYPES; q++)
      if (q == sp) o = off[q];
    spos[k] = ((v & 0xffff) + o) | (sp << 16);
  }
  __syncwarp();
}

template <class T>
__device__ __forceinline__ void record_slot(const RowSink& sk, size_t row, int nr, int pos, int j,
                                            const SlotVals<T>& sv) {
  typedef typename Vec4<T>::type T4;
  unsigned char* rec = static_cast<unsigned char*>(sk.rows) + row * (size_t)sk.stride;
  T4 u, v;
  u.x = sv.ux; u.y = sv.uy; u.z = sv.uz; u.w = sv.fc;
  v.x = sv.rinv; v.y = sv.dfc; v.z = sv.d; v.w = sv.dd;
  reinterpret_cast<T4*>(rec)[pos] = u;
  reinterpret_cast<T4*>(rec + row_off_v(nr, (int)sizeof(T)))[pos] = v;
  reinterpret_cast<int*>(rec + row_off_id(nr, (int)sizeof(T)))[pos] = j;
}

// header of a record: n, m, neighbours per species, angular neighbours per species (the first nang slots of the
// distance-sorted row are the angular ones); one warp, after every slot has been written
__device__ __forceinline__ void record_header(const RowSink& sk, size_t row, int nr, int es, const int* spos, int n,
                                              int nang, const int (&cnt)[STAFB_MAX_TYPES], int lane) {
  int ca[STAFB_MAX_TYPES];
#pragma unroll
  for (int q = 0; q < STAFB_MAX_TYPES; q++) ca[q] = 0;
  for (int k0 = 0; k0 < nang; k0 += 32) {
    const int k = k0 + lane;
    const int sp = (k < nang) ? (spos[k] >> 16) : -1;
#pragma unroll
    for (int q = 0; q < STAFB_MAX_TYPES; q++) ca[q] += __popc(__ballot_sync(0xffffffffu, sp == q));
  }
  if (lane == 0) {
    int* h = reinterpret_cast<int*>(static_cast<unsigned char*>(sk.rows) + row * (size_t)sk.stride +
                                    row_off_hdr(nr, es));
    h[0] = n;
    h[1] = nang;
#pragma unroll
    for (int q = 0; q < STAFB_MAX_TYPES; q++) { h[2 + q] = cnt[q]; h[6 + q] = ca[q]; }
    h[10] = 0; h[11] = 0;
  }
}

// One warp per central atom: candidate discovery over the 27 neighbour cells in the
// reference's visiting order (x outer, y, z inner, offsets -1,0,1: celle_gpu.cu.cc:61-82),
// stable sort by dist2 (celle_gpu.cu.cc:128-152), then the radial descriptor row
// (reforce.cu.cc:17-110).
template <class T, int WARPS>
__global__ void __launch_bounds__(WARPS * 32)
    k_nl_radial(int nf, int N, int ncen, int nr, CoreCoef<T> cc, const FrameGeom<T>* __restrict__ fg,
                const T* __restrict__ frac, const int* __restrict__ cell_of, const int* __restrict__ cell_start,
                const int* __restrict__ cells_sorted, int cell_cap, T* __restrict__ raddescr,
                T* __restrict__ des3bsupp, int* __restrict__ intmap2b, T* __restrict__ der2b,
                T* __restrict__ der3bsupp, int* __restrict__ numtriplet, T* __restrict__ geom, T* __restrict__ gsc,
                int na, int* __restrict__ status, RowSink sink) {
  extern __shared__ unsigned char smem_raw[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int gi = blockIdx.x * WARPS + warp;  // row index: the centres are the first ncen atoms of each frame
  if (gi >= nf * ncen) return;
  chain_wait();  // the cell lists come from the kernel just before this one
  const int b = gi / ncen, i = gi - b * ncen;
  // per-warp rows: d2a[nr] d2b[nr] (T) then ja[nr] jb[nr] (int)
  T* d2a = reinterpret_cast<T*>(smem_raw) + (size_t)warp * 2 * nr;
  T* d2b = d2a + nr;
  int* ja = reinterpret_cast<int*>(reinterpret_cast<T*>(smem_raw) + (size_t)WARPS * 2 * nr) + (size_t)warp * 2 * nr;
  int* jb = ja + nr;

  const FrameGeom<T> g = fg[b];
  const T* fr = frac + (size_t)b * N * 3;
  const T pix = fr[3 * i], piy = fr[3 * i + 1], piz = fr[3 * i + 2];
  const int ci = cell_of[(size_t)b * N + i];
  const int cz = ci / (g.nx * g.ny), rem = ci - cz * (g.nx * g.ny), cy = rem / g.nx, cx = rem - cy * g.nx;
  const int* cst = cell_start + (size_t)b * (cell_cap + 1);
  const int* cl = cells_sorted + (size_t)b * N;
  const T cut2 = cc.Rc * cc.Rc;
  const unsigned lt = (1u << lane) - 1u;
  // The 27 neighbour cells in the reference's visiting order, flattened into one candidate list so
  // that all 32 lanes work on every pass: lane q < 27 owns cell q, an inclusive scan gives each cell's
  // offset in the list, and a candidate finds its cell by bisection.
  int* cbeg = reinterpret_cast<int*>(reinterpret_cast<int*>(reinterpret_cast<T*>(smem_raw) + (size_t)WARPS * 2 * nr) +
                                     (size_t)WARPS * 2 * nr) + warp * 64;  // [32] cell starts, [32] list offsets
  int* coff = cbeg + 32;
  {
    int s0 = 0, cn = 0;
    if (lane < 27) {
      const int di = lane / 9 - 1, dj = (lane / 3) % 3 - 1, dk = lane % 3 - 1;
      int bi = cx + di, bj = cy + dj, bk = cz + dk;
      if (bi < 0) bi = g.nx - 1; else if (bi == g.nx) bi = 0;
      if (bj < 0) bj = g.ny - 1; else if (bj == g.ny) bj = 0;
      if (bk < 0) bk = g.nz - 1; else if (bk == g.nz) bk = 0;
      const int c = bi + bj * g.nx + bk * g.nx * g.ny;
      s0 = cst[c];
      cn = cst[c + 1] - s0;
    }
    int x = cn;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int y = __shfl_up_sync(0xffffffffu, x, o);
      if (lane >= o) x += y;
    }
    cbeg[lane] = s0;
    coff[lane] = x - cn;  // exclusive offset; lanes >= 27 hold the total
  }
  __syncwarp();
  const int M = coff[27];
  int count = 0;
  for (int e0 = 0; e0 < M; e0 += 32) {
    const int e = e0 + lane;
    bool pred = false;
    int j = -1;
    T dist2 = T(0);
    if (e < M) {
      int q = 0;
#pragma unroll
      for (int st = 16; st > 0; st >>= 1)
        if (q + st < 27 && coff[q + st] <= e) q += st;
      j = cl[cbeg[q] + (e - coff[q])];
      T dx, dy, dz;
      mic_vec(g, fr[3 * j], fr[3 * j + 1], fr[3 * j + 2], pix, piy, piz, dx, dy, dz);
      dist2 = dx * dx + dy * dy + dz * dz;
      pred = (dist2 < cut2) && (j != i);
    }
    const unsigned bal = __ballot_sync(0xffffffffu, pred);
    const int slot = count + __popc(bal & lt);
    if (pred && slot < nr) {
      d2a[slot] = dist2;
      ja[slot] = j;
    }
    count += __popc(bal);
  }
  if (count > nr && lane == 0) set_status(status, STAFB_ERR_RADIAL_OVERFLOW);
  const int n = count < nr ? count : nr;
  __syncwarp();
  // stable rank sort: position = #{f : d2[f] < d2[e] or (equal and f < e)}
  for (int e = lane; e < n; e += 32) {
    const T key = d2a[e];
    int r = 0;
    for (int f = 0; f < n; f++) {
      const T kf = d2a[f];
      r += (kf < key) || (kf == key && f < e);
    }
    d2b[r] = key;
    jb[r] = ja[e];
  }
  __syncwarp();
  const size_t base = (size_t)gi;
  int cnt[STAFB_MAX_TYPES];
  if (sink.rows) group_by_species(sink, jb, n, lane, ja, cnt);  // ja[] is free after the sort
  int nang = 0;
  for (int k = lane; k < nr; k += 32) {
    T vx = T(0), vy = T(0), vz = T(0);
    int j = 0;
    if (k < n) {
      j = jb[k];
      mic_vec(g, pix, piy, piz, fr[3 * j], fr[3 * j + 1], fr[3 * j + 2], vx, vy, vz);
    }
    SlotVals<T> sv;
    radial_slot<T>(cc, k < n, j, vx, vy, vz, base, k, nr, raddescr, des3bsupp, intmap2b, der2b, der3bsupp, geom, gsc,
                   nang, sv);
    if (sink.rows && k < n) record_slot<T>(sink, base, nr, ja[k] & 0xffff, j, sv);
  }
  nang = warp_sum(nang);
  if (sink.rows) record_header(sink, base, nr, (int)sizeof(T), ja, n, nang, cnt, lane);
  if (lane == 0) {
    if (intmap2b) intmap2b[base * (nr + 1)] = n;
    if (numtriplet) numtriplet[base] = nang;
    if ((long long)nang * (nang - 1) / 2 > na) set_status(status, STAFB_ERR_ANGULAR_OVERFLOW);
  }
}

// Radial rows from a caller-supplied neighbour list: the contract LAMMPS drives libstaf with
// (libstaf/src/staf_api.cpp:304-347, libstaf/vendor/jmd/nn_nn_mlp.cu:174-206,847-853).  The rows are
// already cutoff-filtered and distance-sorted by the caller and ghost atoms carry their periodic image,
// so there is no search, no sort and no minimum-image wrap: v = r_i - r_j in Cartesian space.
// One warp per centre; the centres are the first ncen of the nall atoms.
template <class T, int WARPS>
__global__ void __launch_bounds__(WARPS * 32)
    k_rows_from_list(int ncen, int nall, int nr, CoreCoef<T> cc, const T* __restrict__ pos,
                     const int* __restrict__ howmany, const int* __restrict__ with, int na, int* __restrict__ status,
                     RowSink sink) {
  extern __shared__ unsigned char smem_raw[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int i = blockIdx.x * WARPS + warp;
  if (i >= ncen) return;
  int* ids = reinterpret_cast<int*>(smem_raw) + (size_t)warp * 2 * nr;  // [nr] neighbour of slot k (0 if invalid)
  int* spos = ids + nr;                                                 // [nr] position in the record | species << 16
  int n = howmany[i];
  if (n < 0) n = 0;
  if (n > nr) {
    if (lane == 0) set_status(status, STAFB_ERR_RADIAL_OVERFLOW);
    n = nr;
  }
  // a bad entry (out of range or the centre itself) is reported and dropped: the row is compacted first
  int nv = 0;
  const unsigned lt = (1u << lane) - 1u;
  for (int k0 = 0; k0 < n; k0 += 32) {
    const int k = k0 + lane;
    int j = -1;
    if (k < n) {
      j = with[(size_t)i * nr + k];
      if (j < 0 || j >= nall || j == i) {
        set_status(status, STAFB_ERR_INVALID);
        j = -1;
      }
    }
    const unsigned bal = __ballot_sync(0xffffffffu, j >= 0);
    if (j >= 0) ids[nv + __popc(bal & lt)] = j;
    nv += __popc(bal);
  }
  n = nv;
  __syncwarp();
  const T pix = pos[3 * i], piy = pos[3 * i + 1], piz = pos[3 * i + 2];
  const size_t base = (size_t)i;
  int cnt[STAFB_MAX_TYPES];
  group_by_species(sink, ids, n, lane, spos, cnt);
  int nang = 0;
  for (int k = lane; k < n; k += 32) {
    const int j = ids[k];
    SlotVals<T> sv;
    radial_slot<T>(cc, true, j, pix - pos[3 * j], piy - pos[3 * j + 1], piz - pos[3 * j + 2], base, k, nr,
                   (T*)nullptr, (T*)nullptr, (int*)nullptr, (T*)nullptr, (T*)nullptr, (T*)nullptr, (T*)nullptr, nang,
                   sv);
    record_slot<T>(sink, base, nr, spos[k] & 0xffff, j, sv);
  }
  nang = warp_sum(nang);
  record_header(sink, base, nr, (int)sizeof(T), spos, n, nang, cnt, lane);
  if (lane == 0 && (long long)nang * (nang - 1) / 2 > na) set_status(status, STAFB_ERR_ANGULAR_OVERFLOW);
}

// Angular descriptor rows (reforce.cu.cc:112-236): one block per central atom; the sorted
// neighbour geometry is staged in shared memory and the block writes the three angular
// tensors with consecutive threads on consecutive triplet slots.
template <class T, int THREADS>
__global__ void __launch_bounds__(THREADS)
    k_angular(int nf, int N, int nr, int na, T Ra, const T* __restrict__ geom, const int* __restrict__ intmap2b,
              const int* __restrict__ numtriplet, T* __restrict__ angdescr, int* __restrict__ intmap3b,
              T* __restrict__ der3b) {
  extern __shared__ unsigned char smem_raw[];
  typedef typename Vec4<T>::type T4;
  typedef typename Vec2<T>::type T2;
  T4* v = reinterpret_cast<T4*>(smem_raw);             // [nr] vector + norm
  T* fc = reinterpret_cast<T*>(v + nr);                // [nr] cutoff
  T* dcp = fc + nr;                                    // [nr] dc prefactor
  int* ids = reinterpret_cast<int*>(dcp + nr);         // [nr]
  const size_t base = blockIdx.x;
  int m = numtriplet[base];
  if (m > nr) m = nr;
  const T PI = PIc<T>();
  for (int k = threadIdx.x; k < m; k += THREADS) {
    T4 q = reinterpret_cast<const T4*>(geom)[base * nr + k];
    v[k] = q;
    fc[k] = T(0.5) * (T(1.) + r_cos(PI * q.w / Ra));
    dcp[k] = -T(0.5) * r_sin(PI * q.w / Ra) * PI / Ra / q.w;
    ids[k] = intmap2b[base * (nr + 1) + 1 + k];
  }
  __syncthreads();
  long long Tl = (long long)m * (m - 1) / 2;
  const int Tn = Tl < na ? (int)Tl : na;
  int2* im3 = reinterpret_cast<int2*>(intmap3b) + base * na;
  T* ad = angdescr + base * na;
  T2* d3x = reinterpret_cast<T2*>(der3b) + (base * 3 + 0) * na;
  T2* d3y = reinterpret_cast<T2*>(der3b) + (base * 3 + 1) * na;
  T2* d3z = reinterpret_cast<T2*>(der3b) + (base * 3 + 2) * na;
  for (int nn = threadIdx.x; nn < na; nn += THREADS) {
    T t = T(0);
    int2 id = make_int2(0, 0);
    T2 ox, oy, oz;
    ox.x = ox.y = oy.x = oy.y = oz.x = oz.y = T(0);
    if (nn < Tn) {
      int j, k;
      unrank_pair(nn, m, j, k);
      const T4 a = v[j], c = v[k];
      const T cj = fc[j], ck = fc[k];
      const T dot = a.x * c.x + a.y * c.y + a.z * c.z;
      const T angle = dot / (a.w * c.w);
      const T half = T(0.5) * (angle + T(1));
      t = half * cj * ck;
      const T dj3 = a.w * a.w * a.w * c.w, dk3 = c.w * c.w * c.w * a.w;
      const T nj2 = a.w * a.w, nk2 = c.w * c.w;
      const T pj = dcp[j], pk = dcp[k];
      ox.x = (T(0.5) * (nj2 * c.x - a.x * dot) / dj3) * cj * ck + half * (pj * a.x) * ck;
      ox.y = (T(0.5) * (nk2 * a.x - c.x * dot) / dk3) * cj * ck + half * cj * (pk * c.x);
      oy.x = (T(0.5) * (nj2 * c.y - a.y * dot) / dj3) * cj * ck + half * (pj * a.y) * ck;
      oy.y = (T(0.5) * (nk2 * a.y - c.y * dot) / dk3) * cj * ck + half * cj * (pk * c.y);
      oz.x = (T(0.5) * (nj2 * c.z - a.z * dot) / dj3) * cj * ck + half * (pj * a.z) * ck;
      oz.y = (T(0.5) * (nk2 * a.z - c.z * dot) / dk3) * cj * ck + half * cj * (pk * c.z);
      id = make_int2(ids[j], ids[k]);
    }
    ad[nn] = t;
    im3[nn] = id;
    d3x[nn] = ox;
    d3y[nn] = oy;
    d3z[nn] = oz;
  }
}

template <class T>
int launch_descriptors(stafb_ctx* c, cudaStream_t s, const T* pos, const T* box, int nf, int N, T* raddescr,
                       T* angdescr, T* des3bsupp, int* intmap2b, int* intmap3b, T* der2b, T* der3b, T* der3bsupp,
                       int* numtriplet, int ncen, const RowSink* sink) {
  if (nf <= 0 || N <= 0) return STAFB_ERR_INVALID;
  if (nf > c->max_batch || N > c->n_max) return STAFB_ERR_CAPACITY;
  if (ncen < 0) ncen = N;  // every atom is a centre unless the caller restricts the rows to the first ncen
  if (ncen > N) return STAFB_ERR_INVALID;
  const int nr = c->nr, na = c->na, cap = c->cell_cap;
  FrameGeom<T>* fg = reinterpret_cast<FrameGeom<T>*>(c->fgeom);
  T* frac = reinterpret_cast<T*>(c->frac);
  // the compact geometry rows feed the angular-descriptor kernel only
  const bool want_angular = angdescr && intmap3b && der3b;
  T* geom = want_angular ? reinterpret_cast<T*>(c->geom) : nullptr;
  T* gsc = want_angular ? reinterpret_cast<T*>(c->gsc) : nullptr;
  RowSink sk;
  memset(&sk, 0, sizeof(sk));
  if (sink) sk = *sink;
  if (want_angular && (!intmap2b || !numtriplet)) return STAFB_ERR_INVALID;
  int mpc = N / 3;  // descriptor_builder/reforce.cc:306-309
  if (mpc < 1) mpc = 1;
  if (mpc > 256) mpc = 256;
  CoreCoef<T> cc;
  cc.Rc = (T)c->Rc; cc.Rs = (T)c->Rs; cc.Ra = (T)c->Ra;
  cc.A = (T)c->coef[0]; cc.B = (T)c->coef[1]; cc.C = (T)c->coef[2]; cc.pa = (T)c->coef[3]; cc.pb = (T)c->coef[4];
  const int tot = nf * N;
  const size_t small_sm = sizeof(int) * ((size_t)cap + 1 + N);
  if (small_sm <= 48 * 1024 && N <= 2048) {
    k_cell_lists_small<T><<<nf, 1024, small_sm, s>>>(pos, box, N, cc.Rc, cap, mpc, fg, frac, c->cell_of, c->cell_start,
                                                    c->cells_sorted, c->status_d);
    c->launches += 1;
  } else {
    STAFB_CUDA_OK(cudaMemsetAsync(c->cell_count, 0, sizeof(int) * (size_t)nf * cap, s));
    // each of these needs all of its predecessor's output: chained launches only save the launch gaps
    STAFB_CUDA_OK(launch_chained(k_cells<T>, dim3((N + 255) / 256, nf), 256, 0, s, pos, box, nf, N, cc.Rc, cap, fg,
                                 frac, c->cell_of, c->cell_count, c->status_d));
    STAFB_CUDA_OK(launch_chained(k_scan<T>, nf, 1024, 0, s, (const FrameGeom<T>*)fg, (const int*)c->cell_count,
                                 c->cell_start, c->cell_cursor, cap, mpc, c->status_d));
    const long long warps = (long long)nf * cap;
    if (N <= 4096) {
      STAFB_CUDA_OK(launch_chained(k_gather_cells<T>, (unsigned)((warps * 32 + 255) / 256), 256, 0, s,
                                   (const FrameGeom<T>*)fg, nf, N, (const int*)c->cell_of, (const int*)c->cell_start,
                                   c->cells_sorted, cap));
      c->launches += 4;
    } else {
      STAFB_CUDA_OK(launch_chained(k_fill, (tot + 255) / 256, 256, 0, s, nf, N, (const int*)c->cell_of,
                                   (const int*)c->cell_start, c->cell_cursor, c->cells_raw, cap));
      STAFB_CUDA_OK(launch_chained(k_sort_cells<T>, (unsigned)((warps * 32 + 255) / 256), 256, 0, s,
                                   (const FrameGeom<T>*)fg, nf, N, (const int*)c->cell_start, (const int*)c->cells_raw,
                                   c->cells_sorted, cap));
      c->launches += 5;
    }
  }
  {
    constexpr int W = 4;
    size_t sm = (size_t)W * 2 * nr * (sizeof(T) + sizeof(int)) + (size_t)W * 64 * sizeof(int);
    const int rows = nf * ncen;
    STAFB_CUDA_OK(launch_chained(k_nl_radial<T, W>, (rows + W - 1) / W, W * 32, sm, s, nf, N, ncen, nr, cc, fg, frac,
                                 c->cell_of, c->cell_start, c->cells_sorted, cap, raddescr, des3bsupp, intmap2b, der2b,
                                 der3bsupp, numtriplet, geom, gsc, na, c->status_d, sk));
  }
  c->launches += 1;
  if (want_angular) {
    constexpr int TH = 128;
    size_t sm = (size_t)nr * (sizeof(typename Vec4<T>::type) + 2 * sizeof(T) + sizeof(int));
    k_angular<T, TH><<<nf * ncen, TH, sm, s>>>(nf, N, nr, na, cc.Ra, geom, intmap2b, numtriplet, angdescr, intmap3b, der3b);
    c->launches += 1;
  }
  STAFB_CUDA_OK(cudaGetLastError());
  return STAFB_OK;
}

template int launch_descriptors<float>(stafb_ctx*, cudaStream_t, const float*, const float*, int, int, float*, float*,
                                       float*, int*, int*, float*, float*, float*, int*, int, const RowSink*);
template int launch_descriptors<double>(stafb_ctx*, cudaStream_t, const double*, const double*, int, int, double*,
                                        double*, double*, int*, int*, double*, double*, double*, int*, int,
                                        const RowSink*);

template <class T>
int launch_rows_from_list(stafb_ctx* c, cudaStream_t s, const T* pos, int ncen, int nall, const int* howmany,
                          const int* with, const RowSink* sink) {
  if (ncen <= 0 || nall < ncen || !howmany || !with || !sink || !sink->rows) return STAFB_ERR_INVALID;
  if (nall > c->n_max) return STAFB_ERR_CAPACITY;
  CoreCoef<T> cc;
  cc.Rc = (T)c->Rc; cc.Rs = (T)c->Rs; cc.Ra = (T)c->Ra;
  cc.A = (T)c->coef[0]; cc.B = (T)c->coef[1]; cc.C = (T)c->coef[2]; cc.pa = (T)c->coef[3]; cc.pb = (T)c->coef[4];
  constexpr int W = 4;
  const size_t sm = (size_t)W * 2 * c->nr * sizeof(int);
  k_rows_from_list<T, W><<<(ncen + W - 1) / W, W * 32, sm, s>>>(ncen, nall, c->nr, cc, pos, howmany, with, c->na,
                                                              c->status_d, *sink);
  c->launches += 1;
  STAFB_CUDA_OK(cudaGetLastError());
  return STAFB_OK;
}
template int launch_rows_from_list<float>(stafb_ctx*, cudaStream_t, const float*, int, int, const int*, const int*,
                                          const RowSink*);
template int launch_rows_from_list<double>(stafb_ctx*, cudaStream_t, const double*, int, int, const int*, const int*,
                                           const RowSink*);

}  // namespace stafb

// ---------------------------------------------------------------------------------------------
// ComputeDescriptorsLight without any allocation.
//
// Some callers cannot allocate device memory at the point where they need the descriptors: code
// running inside a framework's op callback whose memory is owned by that framework's allocator, a
// plug-in invoked while another library holds the allocator lock, or a process that was given a fixed
// memory budget up front.  stafb_create() calls cudaMalloc for the neighbour-list scratch (fractional
// coordinates, the cell lists, the sorted neighbour rows); this entry point keeps that scratch in a
// fixed array that is part of the library image instead.  Every GPU that loads the library holds those
// STAFB_NOALLOC_SCRATCH_BYTES until the process exits.
//
// Limits: nf*N <= 1024 atoms per call, nf <= 16 frames, radial_buffer <= 64.  All calls share the one
// array, so two calls that overlap on the same GPU (different streams or threads) race; the array keeps
// the previous call's contents, and the parts that must start at zero (cell counters, status word) are
// cleared on the stream at the start of every call.
namespace {
constexpr int NOALLOC_MAX_ATOMS = 1024;
constexpr int NOALLOC_MAX_FRAMES = 16;
constexpr int NOALLOC_MAX_NR = 64;
constexpr int NOALLOC_MAX_CELLS = 4 * NOALLOC_MAX_ATOMS + 64 * NOALLOC_MAX_FRAMES + 27 * 4 * NOALLOC_MAX_FRAMES;
constexpr size_t al256(size_t x) { return (x + 255) & ~(size_t)255; }
constexpr size_t NA_OFF_FGEOM = 0;
constexpr size_t NA_OFF_FRAC = NA_OFF_FGEOM + al256(sizeof(stafb::FrameGeom<double>) * NOALLOC_MAX_FRAMES);
constexpr size_t NA_OFF_CELLOF = NA_OFF_FRAC + al256(sizeof(double) * 3 * NOALLOC_MAX_ATOMS);
constexpr size_t NA_OFF_COUNT = NA_OFF_CELLOF + al256(sizeof(int) * NOALLOC_MAX_ATOMS);
constexpr size_t NA_OFF_START = NA_OFF_COUNT + al256(sizeof(int) * NOALLOC_MAX_CELLS);
constexpr size_t NA_OFF_CURSOR = NA_OFF_START + al256(sizeof(int) * (NOALLOC_MAX_CELLS + NOALLOC_MAX_FRAMES));
constexpr size_t NA_OFF_RAW = NA_OFF_CURSOR + al256(sizeof(int) * NOALLOC_MAX_CELLS);
constexpr size_t NA_OFF_SORTED = NA_OFF_RAW + al256(sizeof(int) * NOALLOC_MAX_ATOMS);
constexpr size_t NA_OFF_GEOM = NA_OFF_SORTED + al256(sizeof(int) * NOALLOC_MAX_ATOMS);
constexpr size_t NA_OFF_GSC = NA_OFF_GEOM + al256(sizeof(double) * 4 * NOALLOC_MAX_ATOMS * NOALLOC_MAX_NR);
constexpr size_t NA_OFF_STATUS = NA_OFF_GSC + al256(sizeof(double) * 2 * NOALLOC_MAX_ATOMS * NOALLOC_MAX_NR);
constexpr size_t NA_TOTAL = NA_OFF_STATUS + 256;
constexpr int NOALLOC_MAX_DEVICES = 64;
}  // namespace

// The scratch itself.  In host code this name is only a handle for cudaGetSymbolAddress; the device
// address is looked up once per device below.
static __device__ __align__(256) unsigned char g_noalloc_scratch[NA_TOTAL];
static void* g_noalloc_addr[NOALLOC_MAX_DEVICES] = {nullptr};

extern "C" size_t stafb_noalloc_scratch_bytes(void) { return NA_TOTAL; }

extern "C" int stafb_compute_descriptors_light_noalloc(int dtype, double radial_cutoff, double rs, double ra,
                                                       int radial_buffer, int angular_buffer, void* stream,
                                                       const void* positions_d, const void* boxer_d, int nf, int N,
                                                       void* raddescr_d, void* angdescr_d, void* des3bsupp_d,
                                                       int* intmap2b_d, int* intmap3b_d, void* der2b_d,
                                                       void* der3b_d, void* der3bsupp_d, int* numtriplet_d,
                                                       int* status_out_d) {
  if ((dtype != STAFB_F32 && dtype != STAFB_F64) || !positions_d || !boxer_d || !raddescr_d || !des3bsupp_d ||
      !intmap2b_d || !der2b_d || !der3bsupp_d || !numtriplet_d || nf <= 0 || N <= 0 || radial_buffer <= 0 ||
      angular_buffer <= 0 || !(radial_cutoff > 0) || !(ra > 0) || ra > radial_cutoff)
    return STAFB_ERR_INVALID;
  if (nf > NOALLOC_MAX_FRAMES || (long long)nf * N > NOALLOC_MAX_ATOMS || radial_buffer > NOALLOC_MAX_NR) {
    fprintf(stderr,
            "stafb_compute_descriptors_light_noalloc: nf=%d N=%d radial_buffer=%d exceed the built-in scratch "
            "(at most %d frames, %d atoms in total, radial_buffer %d); use stafb_create + "
            "stafb_compute_descriptors_light\n",
            nf, N, radial_buffer, NOALLOC_MAX_FRAMES, NOALLOC_MAX_ATOMS, NOALLOC_MAX_NR);
    return STAFB_ERR_CAPACITY;
  }
  const int cell_cap = 4 * (N > 27 ? N : 27) + 64;
  if ((long long)nf * cell_cap > NOALLOC_MAX_CELLS) return STAFB_ERR_CAPACITY;
  int dev = 0;
  STAFB_CUDA_OK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= NOALLOC_MAX_DEVICES) return STAFB_ERR_CAPACITY;
  if (!g_noalloc_addr[dev]) {
    // first call on this device (do it before any stream capture): resolve the device address of the array.
    // Two threads making their first call together both store the same value; no lock is needed for that.
    void* p = nullptr;
    STAFB_CUDA_OK(cudaGetSymbolAddress(&p, g_noalloc_scratch));
    g_noalloc_addr[dev] = p;
  }
  unsigned char* base = static_cast<unsigned char*>(g_noalloc_addr[dev]);
  cudaStream_t s = (cudaStream_t)stream;
  stafb_ctx c;
  memset(&c, 0, sizeof(c));
  c.dtype = dtype;
  c.Rc = radial_cutoff; c.Rs = rs; c.Ra = ra;
  c.nr = radial_buffer; c.na = angular_buffer; c.n_max = N; c.max_batch = nf;
  stafb_core_coefficients_for(dtype, radial_cutoff, rs, c.coef);
  c.device = dev;
  c.cell_cap = cell_cap;
  c.fgeom = base + NA_OFF_FGEOM;
  c.frac = base + NA_OFF_FRAC;
  c.cell_of = reinterpret_cast<int*>(base + NA_OFF_CELLOF);
  c.cell_count = reinterpret_cast<int*>(base + NA_OFF_COUNT);
  c.cell_start = reinterpret_cast<int*>(base + NA_OFF_START);
  c.cell_cursor = reinterpret_cast<int*>(base + NA_OFF_CURSOR);
  c.cells_raw = reinterpret_cast<int*>(base + NA_OFF_RAW);
  c.cells_sorted = reinterpret_cast<int*>(base + NA_OFF_SORTED);
  c.geom = base + NA_OFF_GEOM;
  c.gsc = base + NA_OFF_GSC;
  c.status_d = reinterpret_cast<int*>(base + NA_OFF_STATUS);
  // the shared array keeps the previous call's contents: clear the status word here (the cell
  // counters are cleared by the descriptor launch sequence itself)
  STAFB_CUDA_OK(cudaMemsetAsync(c.status_d, 0, sizeof(int), s));
  int rc;
  if (dtype == STAFB_F32)
    rc = stafb::launch_descriptors<float>(&c, s, (const float*)positions_d, (const float*)boxer_d, nf, N,
                                          (float*)raddescr_d, (float*)angdescr_d, (float*)des3bsupp_d, intmap2b_d,
                                          intmap3b_d, (float*)der2b_d, (float*)der3b_d, (float*)der3bsupp_d,
                                          numtriplet_d);
  else
    rc = stafb::launch_descriptors<double>(&c, s, (const double*)positions_d, (const double*)boxer_d, nf, N,
                                           (double*)raddescr_d, (double*)angdescr_d, (double*)des3bsupp_d,
                                           intmap2b_d, intmap3b_d, (double*)der2b_d, (double*)der3b_d,
                                           (double*)der3bsupp_d, numtriplet_d);
  if (rc != STAFB_OK) return rc;
  if (status_out_d)
    STAFB_CUDA_OK(cudaMemcpyAsync(status_out_d, c.status_d, sizeof(int), cudaMemcpyDeviceToDevice, s));
  return STAFB_OK;
}
