// Shared device helpers and host-side handle layouts of the stafb library (sm_100a).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include "../../include/stafb.h"

namespace stafb {

// The reference uses this literal, not pi (STAF/src/descriptor_builder/reforce.cu.cc:15).
template <class T> __host__ __device__ __forceinline__ T PIc() { return T(3.141592654); }

template <class T> struct Vec2;
template <> struct Vec2<float> { typedef float2 type; };
template <> struct Vec2<double> { typedef double2 type; };
template <class T> struct Vec4;
template <> struct Vec4<float> { typedef float4 type; };
template <> struct Vec4<double> { typedef double4 type; };

__device__ __forceinline__ float r_exp(float x) { return expf(x); }
__device__ __forceinline__ double r_exp(double x) { return exp(x); }
__device__ __forceinline__ float r_log(float x) { return logf(x); }
__device__ __forceinline__ double r_log(double x) { return log(x); }
__device__ __forceinline__ float r_tanh(float x) { return tanhf(x); }
__device__ __forceinline__ double r_tanh(double x) { return tanh(x); }
__device__ __forceinline__ float r_cos(float x) { return cosf(x); }
__device__ __forceinline__ double r_cos(double x) { return cos(x); }
__device__ __forceinline__ float r_sin(float x) { return sinf(x); }
__device__ __forceinline__ double r_sin(double x) { return sin(x); }
__device__ __forceinline__ float r_sqrt(float x) { return sqrtf(x); }
__device__ __forceinline__ double r_sqrt(double x) { return sqrt(x); }
__device__ __forceinline__ float r_pow(float x, float y) { return powf(x, y); }
__device__ __forceinline__ double r_pow(double x, double y) { return pow(x, y); }
__device__ __forceinline__ float r_rint(float x) { return rintf(x); }
__device__ __forceinline__ double r_rint(double x) { return rint(x); }
__device__ __forceinline__ float r_floor(float x) { return floorf(x); }
__device__ __forceinline__ double r_floor(double x) { return floor(x); }
__device__ __forceinline__ float r_abs(float x) { return fabsf(x); }
__device__ __forceinline__ double r_abs(double x) { return fabs(x); }

// Device code never traps: problems are recorded once in a status word the host reads.
__device__ __forceinline__ void set_status(int* st, int code) { atomicCAS(st, 0, code); }

// Programmatic dependent launch.  A kernel launched through launch_chained() may become resident while the
// kernel before it on the stream is still running; it must call chain_wait() before it reads anything that
// kernel wrote and before its first global write.  What it does ahead of that (staging of neighbour rows or
// weights that are at least two kernels old, shared-memory set-up) overlaps the predecessor's tail.  chain_wait()
// returns once the predecessor has completed and its writes are visible, and only then lets the NEXT kernel of
// the chain start: so whenever a kernel runs its prologue, everything up to two kernels back has completed.
// Both calls are no-ops for a kernel that was launched the ordinary way.
__device__ __forceinline__ void chain_wait() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

inline bool chained_launches_enabled() {
  static const bool on = getenv("STAFB_NO_CHAINED_LAUNCH") == nullptr;
  return on;
}

template <class... KArgs, class... Args>
inline cudaError_t launch_chained(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s,
                                  Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = chained_launches_enabled() ? 1 : 0;
  cfg.attrs = at;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}

template <class T>
__device__ __forceinline__ T warp_sum(T v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Sum over a block of NW warps; result valid in every thread.  `red` is NW+1 elements of smem.
template <class T, int NW>
__device__ __forceinline__ T block_sum(T v, T* red) {
  v = warp_sum(v);
  if (NW == 1) return v;
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  __syncthreads();
  if (l == 0) red[w] = v;
  __syncthreads();
  T s = T(0);
#pragma unroll
  for (int i = 0; i < NW; i++) s += red[i];
  return s;
}

// Triplet slot nn -> pair (j<k) of sorted-neighbour positions in a row of m angular
// neighbours (row-major upper triangle; reforce.cu.cc:137-146), closed form.
__device__ __forceinline__ void unrank_pair(int nn, int m, int& j, int& k) {
  const float b = 2.0f * m - 1.0f;
  int jj = (int)((b - sqrtf(fmaxf(b * b - 8.0f * nn, 0.0f))) * 0.5f);
  if (jj < 0) jj = 0;
  if (jj > m - 2) jj = m - 2;
  while (jj > 0 && (jj * (2 * m - jj - 1)) / 2 > nn) jj--;
  while (((jj + 1) * (2 * m - jj - 2)) / 2 <= nn) jj++;
  j = jj;
  k = nn - (jj * (2 * m - jj - 1)) / 2 + jj + 1;
}

template <class T>
struct FrameGeom {
  T box[6];
  T inv[6];
  int nx, ny, nz, ncell;
  T sx, sy, sz;
};

template <class T>
struct CoreCoef {
  T Rc, Rs, Ra, A, B, C, pa, pb;
};

// Neighbour record of one central atom, the only thing the fused sweeps read about the geometry.  One
// contiguous block per atom (so that a sweep stages it with a single bulk copy), neighbours grouped by species
// (species 0 first, ...) and distance-sorted inside a group, so that a sweep addresses "the k-th neighbour of
// species q" directly and the angular neighbours (r < Ra) are a prefix of every group:
//   U[nr]   (4 reals)  unit vector (r_i - r_k)/r and the angular cutoff fc(r)
//   V[nr]   (4 reals)  1/r, dfc/dr, radial descriptor d(r), dd/dr
//   id[nr]  (int32)    index of the neighbour in the frame (padded to a multiple of 4 entries)
//   hdr[12] (int32)    n, m = number of angular neighbours, cntR[4] neighbours per species, cntA[4] angular
//                      neighbours per species, 2 unused
// Entries past n are never read.
constexpr int ROW_HDR_INTS = 12;
__host__ __device__ inline int row_off_v(int nr, int es) { return nr * 4 * es; }
__host__ __device__ inline int row_off_id(int nr, int es) { return 2 * nr * 4 * es; }
__host__ __device__ inline int row_off_hdr(int nr, int es) { return 2 * nr * 4 * es + 4 * ((nr + 3) & ~3); }
__host__ __device__ inline int row_stride_bytes(int nr, int es) { return row_off_hdr(nr, es) + 4 * ROW_HDR_INTS; }

// Where the neighbour kernels leave the records, and how they find the species of a neighbour: atoms are
// species-sorted with boundaries shift[] unless a per-atom map is given (owned + ghost atoms of a domain).
struct RowSink {
  void* rows;  // [nf, ncen] records of `stride` bytes; null: no records are written
  int stride;
  int nt;
  int shift[STAFB_MAX_TYPES + 1];
  const int* tmap;
};

}  // namespace stafb

struct stafb_ctx {
  int dtype;
  double Rc, Rs, Ra;
  int nr, na, n_max, max_batch;
  double coef[5];
  int device;
  int cell_cap;  // cells per frame the scratch can hold
  // scratch (device)
  void* fgeom;        // FrameGeom<T>[max_batch]
  void* frac;         // T[max_batch, n_max, 3]
  int* cell_of;       // [max_batch, n_max]
  int* cell_count;    // [max_batch, cell_cap]
  int* cell_start;    // [max_batch, cell_cap+1]
  int* cell_cursor;   // [max_batch, cell_cap]
  int* cells_raw;     // [max_batch, n_max]
  int* cells_sorted;  // [max_batch, n_max]
  void* geom;         // T[max_batch, n_max, nr, 4]: MIC vector r_i - r_j and its norm, sorted order
  void* gsc;          // T[max_batch, n_max, nr, 2]: d(raddescr)/dr and d(des3bsupp)/dr
  int* status_d;
  int* status_h;  // pinned
  int launches;
  // optional per-phase timing of the fused path (CUDA events on the launching stream)
  int timing;
  int n_phase;
  cudaEvent_t ev[16];
};

#define STAFB_CUDA_OK(call)                                        \
  do {                                                             \
    cudaError_t e__ = (call);                                      \
    if (e__ != cudaSuccess) {                                      \
      stafb_record_cuda_error(e__, __FILE__, __LINE__);            \
      return STAFB_ERR_CUDA;                                       \
    }                                                              \
  } while (0)

void stafb_record_cuda_error(cudaError_t e, const char* file, int line);
// repulsive-core coefficients for a dtype (STAFB_F32 / STAFB_F64), evaluated on the host in that precision
void stafb_core_coefficients_for(int dtype, double Rc, double Rs, double out5[5]);

// launchers implemented per translation unit (T = float | double)
namespace stafb {
// The operator outputs (raddescr ... numtriplet) may all be null when only the records of `sink` are wanted.
template <class T>
int launch_descriptors(stafb_ctx* c, cudaStream_t s, const T* pos, const T* box, int nf, int N, T* raddescr,
                       T* angdescr, T* des3bsupp, int* intmap2b, int* intmap3b, T* der2b, T* der3b, T* der3bsupp,
                       int* numtriplet, int ncen = -1, const RowSink* sink = nullptr);
// records of the first ncen atoms from a caller-supplied, distance-sorted neighbour list over nall atoms
template <class T>
int launch_rows_from_list(stafb_ctx* c, cudaStream_t s, const T* pos, int ncen, int nall, const int* howmany,
                          const int* with, const RowSink* sink);
}
