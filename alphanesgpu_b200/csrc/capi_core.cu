// Context management and the descriptor entry point of the C ABI (include/stafb.h).
#include <math.h>
#include <stdlib.h>
#include <string.h>
#include <mutex>
#include <string>
#include "common.cuh"

static std::mutex g_err_mu;
static std::string g_last_cuda_error;

void stafb_record_cuda_error(cudaError_t e, const char* file, int line) {
  std::lock_guard<std::mutex> lk(g_err_mu);
  char buf[512];
  snprintf(buf, sizeof(buf), "%s (%s:%d)", cudaGetErrorString(e), file, line);
  g_last_cuda_error = buf;
}

extern "C" const char* stafb_last_cuda_error(void) {
  std::lock_guard<std::mutex> lk(g_err_mu);
  static thread_local std::string copy;
  copy = g_last_cuda_error;
  return copy.c_str();
}

extern "C" const char* stafb_strerror(int s) {
  switch (s) {
    case STAFB_OK: return "ok";
    case STAFB_ERR_RADIAL_OVERFLOW: return "radial buffer saturated: an atom has more neighbours than radial_buffer";
    case STAFB_ERR_ANGULAR_OVERFLOW: return "angular buffer saturated: m(m-1)/2 exceeds angular_buffer";
    case STAFB_ERR_CELL_OVERFLOW: return "a cell holds more atoms than MAX_PARTICLE_CELLS";
    case STAFB_ERR_BAD_BOX: return "box has a zero length";
    case STAFB_ERR_INVALID: return "invalid argument";
    case STAFB_ERR_CUDA: return "CUDA runtime error";
    case STAFB_ERR_CAPACITY: return "batch, atom count or cell grid exceeds the capacity the context was created with";
    case STAFB_ERR_NONFINITE: return "non-finite result";
    case STAFB_ERR_PEER_TIMEOUT: return "a peer rank did not publish its gradient in time";
    case STAFB_ERR_STAGE_TIMEOUT: return "an asynchronous copy into shared memory did not complete in time";
    default: return "unknown status";
  }
}

// Repulsive-core coefficients A/r^alpha + B/r^beta + C with (alpha,beta) = (1,-30), matched to
// the cosine cutoff in value, first and second derivative at Rs; evaluated in `real` like
// fill_repulsion of STAF/src/descriptor_builder/reforce.cc:101-125.
template <class T>
static void core_coefficients(double Rc, double Rs, double* out) {
  const T PI = T(3.141592654);
  T alpha = 1., beta = -30.;
  T rs = (T)Rs, rc = (T)Rc;
  T f = 0.5 * (cos(PI * rs / rc) + 1);
  T f1 = -0.5 * PI / rc * sin(PI * rs / rc);
  T f2_red = -0.5 * ((PI / rc) * (PI / rc)) * cos(PI * rs / rc) * (rs * rs);
  T gamma_red = 1. / (alpha - beta) * alpha - 1;
  T delta_red = 1. / (alpha - beta) * (f * (alpha - beta) - f1 * rs - f * alpha);
  T eta_red = -alpha / (alpha - beta);
  T epsilon_red = 1. / (alpha - beta) * (rs * f1 + alpha * f);
  T c2_red = alpha * (alpha + 1) * delta_red + beta * (beta + 1) * epsilon_red;
  T c1_red = alpha * (alpha + 1) * gamma_red + beta * (beta + 1) * eta_red;
  T cC = (f2_red - c2_red) / c1_red;
  T eta = -alpha * pow(rs, beta) / (alpha - beta);
  T epsilon = pow(rs, beta) / (alpha - beta) * (rs * f1 + alpha * f);
  T cB = eta * cC + epsilon;
  T gamma = pow(rs, alpha) / (alpha - beta) * alpha - pow(rs, alpha);
  T delta = pow(rs, alpha) / (alpha - beta) * (f * (alpha - beta) - f1 * rs - f * alpha);
  T cA = gamma * cC + delta;
  out[0] = cA; out[1] = cB; out[2] = cC; out[3] = alpha; out[4] = beta;
}

void stafb_core_coefficients_for(int dtype, double Rc, double Rs, double out5[5]) {
  if (dtype == STAFB_F32) core_coefficients<float>(Rc, Rs, out5);
  else core_coefficients<double>(Rc, Rs, out5);
}

extern "C" int stafb_create(stafb_ctx** out, int dtype, double Rc, double Rs, double Ra, int nr, int na, int n_max,
                            int max_batch) {
  if (!out || (dtype != STAFB_F32 && dtype != STAFB_F64) || nr <= 0 || nr > 255 || na <= 0 || n_max <= 0 ||
      max_batch <= 0 || !(Rc > 0) || !(Ra > 0) || Ra > Rc)
    return STAFB_ERR_INVALID;
  stafb_ctx* c = (stafb_ctx*)calloc(1, sizeof(stafb_ctx));
  if (!c) return STAFB_ERR_INVALID;
  c->dtype = dtype;
  c->Rc = Rc; c->Rs = Rs; c->Ra = Ra;
  c->nr = nr; c->na = na; c->n_max = n_max; c->max_batch = max_batch;
  if (dtype == STAFB_F32) core_coefficients<float>(Rc, Rs, c->coef);
  else core_coefficients<double>(Rc, Rs, c->coef);
  STAFB_CUDA_OK(cudaGetDevice(&c->device));
  const size_t es = dtype == STAFB_F32 ? 4 : 8;
  // After the reference's shrink loop the grid has at most max(27, N) cells; the clamp to >= 3 per
  // axis can raise that for very anisotropic boxes, hence the head-room.
  c->cell_cap = 4 * (n_max > 27 ? n_max : 27) + 64;
  const size_t B = (size_t)max_batch, Nn = (size_t)n_max;
  const size_t fg_bytes = dtype == STAFB_F32 ? sizeof(stafb::FrameGeom<float>) : sizeof(stafb::FrameGeom<double>);
  STAFB_CUDA_OK(cudaMalloc(&c->fgeom, fg_bytes * B));
  STAFB_CUDA_OK(cudaMalloc(&c->frac, es * B * Nn * 3));
  STAFB_CUDA_OK(cudaMalloc((void**)&c->cell_of, sizeof(int) * B * Nn));
  STAFB_CUDA_OK(cudaMalloc((void**)&c->cell_count, sizeof(int) * B * c->cell_cap));
  STAFB_CUDA_OK(cudaMalloc((void**)&c->cell_start, sizeof(int) * B * (c->cell_cap + 1)));
  STAFB_CUDA_OK(cudaMalloc((void**)&c->cell_cursor, sizeof(int) * B * c->cell_cap));
  STAFB_CUDA_OK(cudaMalloc((void**)&c->cells_raw, sizeof(int) * B * Nn));
  STAFB_CUDA_OK(cudaMalloc((void**)&c->cells_sorted, sizeof(int) * B * Nn));
  STAFB_CUDA_OK(cudaMalloc(&c->geom, es * B * Nn * nr * 4));
  STAFB_CUDA_OK(cudaMalloc(&c->gsc, es * B * Nn * nr * 2));
  STAFB_CUDA_OK(cudaMalloc((void**)&c->status_d, sizeof(int)));
  STAFB_CUDA_OK(cudaMemset(c->status_d, 0, sizeof(int)));
  STAFB_CUDA_OK(cudaMallocHost((void**)&c->status_h, sizeof(int)));
  *out = c;
  return STAFB_OK;
}

extern "C" void stafb_destroy(stafb_ctx* c) {
  if (!c) return;
  int cur = 0;
  cudaGetDevice(&cur);
  cudaSetDevice(c->device);
  cudaFree(c->fgeom); cudaFree(c->frac); cudaFree(c->cell_of); cudaFree(c->cell_count);
  cudaFree(c->cell_start); cudaFree(c->cell_cursor); cudaFree(c->cells_raw); cudaFree(c->cells_sorted);
  cudaFree(c->geom); cudaFree(c->gsc); cudaFree(c->status_d);
  cudaFreeHost(c->status_h);
  for (int q = 0; q < 16; q++)
    if (c->ev[q]) cudaEventDestroy(c->ev[q]);
  cudaSetDevice(cur);
  free(c);
}

extern "C" int stafb_status(stafb_ctx* c, void* stream) {
  if (!c) return STAFB_ERR_INVALID;
  cudaStream_t s = (cudaStream_t)stream;
  STAFB_CUDA_OK(cudaMemcpyAsync(c->status_h, c->status_d, sizeof(int), cudaMemcpyDeviceToHost, s));
  STAFB_CUDA_OK(cudaMemsetAsync(c->status_d, 0, sizeof(int), s));
  STAFB_CUDA_OK(cudaStreamSynchronize(s));
  return *c->status_h;
}

extern "C" void stafb_core_coefficients(const stafb_ctx* c, double out5[5]) {
  for (int i = 0; i < 5; i++) out5[i] = c->coef[i];
}

extern "C" int stafb_set_phase_timing(stafb_ctx* c, int on) {
  if (!c) return STAFB_ERR_INVALID;
  if (on && !c->ev[0]) {
    for (int q = 0; q < 16; q++) STAFB_CUDA_OK(cudaEventCreate(&c->ev[q]));
  }
  c->timing = on ? 1 : 0;
  c->n_phase = 0;
  return STAFB_OK;
}

extern "C" int stafb_get_phase_times(stafb_ctx* c, float* ms, int cap) {
  if (!c || !ms || !c->timing || c->n_phase < 2) return 0;
  if (cudaEventSynchronize(c->ev[c->n_phase - 1]) != cudaSuccess) return 0;
  int n = c->n_phase - 1;
  if (n > cap) n = cap;
  for (int q = 0; q < n; q++) {
    ms[q] = 0.f;
    cudaEventElapsedTime(&ms[q], c->ev[q], c->ev[q + 1]);
  }
  return n;
}

extern "C" int stafb_last_launch_count(const stafb_ctx* c) { return c ? c->launches : 0; }

extern "C" int stafb_compute_descriptors_light(stafb_ctx* c, void* stream, const void* pos, const void* box, int nf,
                                               int N, void* raddescr, void* angdescr, void* des3bsupp, int* intmap2b,
                                               int* intmap3b, void* der2b, void* der3b, void* der3bsupp,
                                               int* numtriplet) {
  if (!c || !pos || !box || !raddescr || !des3bsupp || !intmap2b || !der2b || !der3bsupp || !numtriplet)
    return STAFB_ERR_INVALID;
  cudaStream_t s = (cudaStream_t)stream;
  c->launches = 0;
  if (c->dtype == STAFB_F32)
    return stafb::launch_descriptors<float>(c, s, (const float*)pos, (const float*)box, nf, N, (float*)raddescr,
                                            (float*)angdescr, (float*)des3bsupp, intmap2b, intmap3b, (float*)der2b,
                                            (float*)der3b, (float*)der3bsupp, numtriplet);
  return stafb::launch_descriptors<double>(c, s, (const double*)pos, (const double*)box, nf, N, (double*)raddescr,
                                           (double*)angdescr, (double*)des3bsupp, intmap2b, intmap3b, (double*)der2b,
                                           (double*)der3b, (double*)der3bsupp, numtriplet);
}

extern "C" int stafb_init_force_radial(int) { return 0; }
extern "C" int stafb_init_force_tripl(int) { return 0; }
extern "C" int stafb_init_grad_force_radial(int) { return 0; }
extern "C" int stafb_init_grad_force_tripl(int) { return 0; }

// ---- measured FP32 / FP64 FMA throughput of the device (the denominator of pipe-utilisation figures) ----
// Every thread runs `iters` rounds of eight independent fused multiply-adds; 2 flops each.
template <class T>
__global__ void __launch_bounds__(256) k_fma_peak(int iters, T seed, T* __restrict__ out) {
  T a0 = seed + threadIdx.x, a1 = a0 + T(1), a2 = a0 + T(2), a3 = a0 + T(3), a4 = a0 + T(4), a5 = a0 + T(5),
    a6 = a0 + T(6), a7 = a0 + T(7);
  const T m = T(0.999), c = T(1e-3);
  for (int i = 0; i < iters; i++) {
    a0 = a0 * m + c; a1 = a1 * m + c; a2 = a2 * m + c; a3 = a3 * m + c;
    a4 = a4 * m + c; a5 = a5 * m + c; a6 = a6 * m + c; a7 = a7 * m + c;
  }
  out[(size_t)blockIdx.x * blockDim.x + threadIdx.x] = a0 + a1 + a2 + a3 + a4 + a5 + a6 + a7;
}

extern "C" int stafb_measure_fma_peak(int dtype, void* stream, double* tflops_out) {
  if (!tflops_out || (dtype != STAFB_F32 && dtype != STAFB_F64)) return STAFB_ERR_INVALID;
  cudaStream_t s = (cudaStream_t)stream;
  int dev = 0, nsm = 0;
  STAFB_CUDA_OK(cudaGetDevice(&dev));
  STAFB_CUDA_OK(cudaDeviceGetAttribute(&nsm, cudaDevAttrMultiProcessorCount, dev));
  const int blocks = nsm * 8, threads = 256, iters = dtype == STAFB_F32 ? 1 << 15 : 1 << 12;
  void* buf = nullptr;
  STAFB_CUDA_OK(cudaMalloc(&buf, (size_t)blocks * threads * 8));
  cudaEvent_t e0, e1;
  STAFB_CUDA_OK(cudaEventCreate(&e0));
  STAFB_CUDA_OK(cudaEventCreate(&e1));
  float best = 1e30f;
  for (int rep = 0; rep < 4; rep++) {  // the first repetition warms up
    cudaEventRecord(e0, s);
    if (dtype == STAFB_F32) k_fma_peak<float><<<blocks, threads, 0, s>>>(iters, 1.0f, (float*)buf);
    else k_fma_peak<double><<<blocks, threads, 0, s>>>(iters, 1.0, (double*)buf);
    cudaEventRecord(e1, s);
    cudaEventSynchronize(e1);
    float ms = 0.f;
    cudaEventElapsedTime(&ms, e0, e1);
    if (rep > 0 && ms < best) best = ms;
  }
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  cudaFree(buf);
  STAFB_CUDA_OK(cudaGetLastError());
  *tflops_out = 2.0 * 8.0 * iters * (double)blocks * threads / (best * 1e-3) / 1e12;
  return STAFB_OK;
}
