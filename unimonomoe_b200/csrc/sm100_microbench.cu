// Hardware micro-benchmarks behind the design decisions of the expert phase of mono_kernel.cu (development tool,
// not part of any library): what one B200 SM sustains for
//   1. scattered row stores (the bf16 partial rows): bytes per clock by contiguous bytes per row per instruction,
//   2. tcgen05.mma kind::f8f6f4 by shape (M = 64 against 128, small N),
//   3. tcgen05.ld 32x32b read-out with 1, 4 and 8 warps,
//   4. cp.async.bulk shared -> global copies by size (would a staged, asynchronous store of partial rows pay?).
// Build and run:  python -m unimonomoe_b200.build microbench  &&  unimonomoe_b200/lib/sm100_microbench
// Every wait in here is bounded by an iteration count.
#include <cuda.h>
#include <cuda_runtime.h>
#include <cstdio>
#include <cstdint>
#include <cstdlib>
#include "ptx_sm100.cuh"
using namespace mono;

#define CK(x) do { cudaError_t e_ = (x); if (e_ != cudaSuccess) { printf("CUDA error %s at %d\n", cudaGetErrorString(e_), __LINE__); exit(1); } } while (0)

// ---------------------------------------------------------------- T1 stores
// Each warp writes `iters` sections of 32 rows x 256 B (rows scattered, 4096 B apart x hash).
template <int MODE>
__global__ void __launch_bounds__(256, 1) store_bench(uint8_t* buf, size_t nrows, int iters, long long* cyc) {
  extern __shared__ uint8_t dyn[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  uint32_t w[8];
  for (int i = 0; i < 8; ++i) w[i] = threadIdx.x * 8 + i;
  const long long t0 = clock64();
  uint32_t h = blockIdx.x * 977u + warp * 131u + 7u;
  for (int it = 0; it < iters; ++it) {
    h = h * 1664525u + 1013904223u;
    const size_t rbase = (static_cast<size_t>(h >> 4) % (nrows / 32)) * 32;   // 32 rows, but scatter them:
    const int colb = (it & 15) * 256;
    if (MODE == 0 || MODE == 4) {          // 16 rows x 64 B per instruction, 8 instructions
      for (int k = 0; k < 8; ++k) {
        const int row = (lane >> 1) + 16 * (k & 1);
        const size_t r = (rbase + row) * 2654435761ull % nrows;
        uint8_t* p = buf + r * 4096 + colb + (k >> 1) * 64 + (lane & 1) * 32;
        if (MODE == 0) st_global_256_stream(p, w); else st_global_256(p, w);
      }
    } else if (MODE == 1) {                // 8 rows x 128 B per instruction
      for (int k = 0; k < 8; ++k) {
        const int row = (lane >> 2) + 8 * (k & 3);
        const size_t r = (rbase + row) * 2654435761ull % nrows;
        uint8_t* p = buf + r * 4096 + colb + (k >> 2) * 128 + (lane & 3) * 32;
        st_global_256_stream(p, w);
      }
    } else if (MODE == 2) {                // 4 rows x 256 B per instruction
      for (int k = 0; k < 8; ++k) {
        const int row = (lane >> 3) + 4 * k;
        const size_t r = (rbase + row) * 2654435761ull % nrows;
        uint8_t* p = buf + r * 4096 + colb + (lane & 7) * 32;
        st_global_256_stream(p, w);
      }
    } else if (MODE == 3) {                // 32 rows x 32 B per instruction
      const size_t r = (rbase + lane) * 2654435761ull % nrows;
      for (int k = 0; k < 8; ++k) {
        uint8_t* p = buf + r * 4096 + colb + k * 32;
        st_global_256_stream(p, w);
      }
    } else if (MODE == 5) {                // 16-byte stores, 4 rows x 128 B per instruction, 16 instructions
      for (int k = 0; k < 16; ++k) {
        const int row = (lane >> 3) + 4 * (k & 7);
        const size_t r = (rbase + row) * 2654435761ull % nrows;
        uint8_t* p = buf + r * 4096 + colb + (k >> 3) * 128 + (lane & 7) * 16;
        asm volatile("st.global.cs.v4.b32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]) : "memory");
      }
    }
  }
  const long long t1 = clock64();
  if (threadIdx.x == 0) cyc[blockIdx.x] = t1 - t0;
}

// ---------------------------------------------------------------- T2 MMA shapes
__global__ void __launch_bounds__(128, 1) mma_bench(int m, int n, int iters, long long* cyc, int* err) {
  extern __shared__ uint8_t dyn_raw[];
  __shared__ uint64_t bar;
  __shared__ uint32_t tmem_slot;
  const uint32_t base = (smem_u32(dyn_raw) + 1023u) & ~1023u;
  uint8_t* dyn = dyn_raw + (base - smem_u32(dyn_raw));
  for (int i = threadIdx.x; i < 48 * 1024 / 4; i += blockDim.x) reinterpret_cast<uint32_t*>(dyn)[i] = 0x38383838u;  // e4m3 1.0
  if (threadIdx.x == 0) { mbar_init(&bar, 1); mbar_init_fence(); }
  if (threadIdx.x < 32) { tmem_alloc(&tmem_slot, 512); tmem_relinquish(); }
  fence_proxy_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tm = tmem_slot;
  if (threadIdx.x == 0) {
    const uint32_t idesc = umma_idesc_e4m3_f32(m, n);
    const uint64_t da = umma_desc_sw128(base), db = umma_desc_sw128(base + 16384);
    const long long t0 = clock64();
    for (int i = 0; i < iters; ++i) {
      const uint32_t d = tm + ((i >> 2) & 1) * 256;   // alternate two accumulators every 4 MMAs, like the kernel
      umma_f8(d, da + 2u * (i & 3), db + 2u * (i & 3), idesc, (i & 3) ? 1u : 0u);
    }
    umma_commit(&bar);
    int spins = 0;
    while (!mbar_try_wait(&bar, 0)) { if (++spins > 20000000) { *err = 1; break; } }
    const long long t1 = clock64();
    cyc[blockIdx.x] = t1 - t0;
  }
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x < 32) { tc_fence_after(); tmem_dealloc(tm, 512); }
}

// ---------------------------------------------------------------- T3 tcgen05.ld rate
template <int COLS>
__global__ void __launch_bounds__(384, 1) tld_bench(int nwarps_active, int iters, long long* cyc, float* sink) {
  extern __shared__ uint8_t dyn_raw[];
  __shared__ uint32_t tmem_slot;
  const int warp = threadIdx.x >> 5;
  if (warp == 0) { tmem_alloc(&tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tm = tmem_slot;
  float acc = 0.f;
  if (warp >= 4 && warp < 4 + nwarps_active) {
    const uint32_t t_lane = tm + (static_cast<uint32_t>((warp & 3) * 32) << 16) + ((warp >= 8) ? 128u : 0u);
    const long long t0 = clock64();
    for (int i = 0; i < iters; ++i) {
      uint32_t v[COLS];
      tmem_ld_n<COLS>(t_lane + (i & 1) * 256, v);
      tmem_ld_wait();
      acc += __uint_as_float(v[0]) + __uint_as_float(v[COLS - 1]);
    }
    const long long t1 = clock64();
    if ((threadIdx.x & 31) == 0) cyc[blockIdx.x * 8 + (warp - 4)] = t1 - t0;
  }
  if (acc == 123.456f) *sink = acc;
  tc_fence_before();
  __syncthreads();
  if (warp == 0) { tc_fence_after(); tmem_dealloc(tm, 512); }
}

// ---------------------------------------------------------------- T4 bulk smem -> global
__global__ void __launch_bounds__(128, 1) bulk_bench(uint8_t* buf, size_t nrows, int bytes, int iters, int lanes, long long* cyc) {
  extern __shared__ uint8_t dyn_raw[];
  const uint32_t base = (smem_u32(dyn_raw) + 1023u) & ~1023u;
  for (int i = threadIdx.x; i < 64 * 1024 / 4; i += blockDim.x) reinterpret_cast<uint32_t*>(dyn_raw + (base - smem_u32(dyn_raw)))[i] = i;
  fence_proxy_async_smem();
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (warp == 0 && lane < lanes) {
    uint32_t h = blockIdx.x * 977u + lane * 131u + 7u;
    const long long t0 = clock64();
    for (int it = 0; it < iters; ++it) {
      h = h * 1664525u + 1013904223u;
      const size_t r = static_cast<size_t>(h >> 4) % nrows;
      uint8_t* g = buf + r * 4096 + (it & 7) * 512;
      const uint32_t s = base + ((lane * bytes) & 0xFFFF);
      asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(g), "r"(s), "r"(bytes) : "memory");
      asm volatile("cp.async.bulk.commit_group;" ::: "memory");
      if ((it & 3) == 3) asm volatile("cp.async.bulk.wait_group.read 2;" ::: "memory");
    }
    asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
    const long long t1 = clock64();
    if (lane == 0) cyc[blockIdx.x] = t1 - t0;
  }
}

static double mean_cyc(long long* d, int n) {
  static long long h[4096];
  CK(cudaMemcpy(h, d, n * sizeof(long long), cudaMemcpyDeviceToHost));
  double s = 0; for (int i = 0; i < n; ++i) s += h[i];
  return s / n;
}

int main() {
  long long* cyc; int* err; float* sink;
  CK(cudaMalloc(&cyc, 4096 * 8)); CK(cudaMalloc(&err, 4)); CK(cudaMalloc(&sink, 4));
  CK(cudaMemset(err, 0, 4));
  const size_t nrows = 131072;   // x 4096 B = 512 MB
  uint8_t* buf; CK(cudaMalloc(&buf, (nrows + 2) * 4096));   // two rows of slack: the widest copy ends 1.5 KB past its row
  const int SM = 200 * 1024;
  cudaEvent_t e0, e1; CK(cudaEventCreate(&e0)); CK(cudaEventCreate(&e1));
#define RUN_STORE(MODE, GRID) do { \
    CK(cudaFuncSetAttribute(store_bench<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, SM)); \
    store_bench<MODE><<<GRID, 256, SM>>>(buf, nrows, 50, cyc); CK(cudaDeviceSynchronize()); \
    const int iters = 400; \
    CK(cudaEventRecord(e0)); store_bench<MODE><<<GRID, 256, SM>>>(buf, nrows, iters, cyc); CK(cudaEventRecord(e1)); CK(cudaDeviceSynchronize()); \
    float ms; CK(cudaEventElapsedTime(&ms, e0, e1)); \
    const double c = mean_cyc(cyc, GRID); const double bytes_sm = 8.0 * iters * 8192; \
    printf("store mode %d grid %3d: %.0f cycles/section/SM  %.1f B/clk/SM  total %.2f TB/s\n", MODE, GRID, c / iters, bytes_sm / c, bytes_sm * GRID / (ms * 1e-3) / 1e12); \
  } while (0)
  for (int g : {8, 148}) {
    if (g == 8) { RUN_STORE(0, 8); RUN_STORE(4, 8); RUN_STORE(1, 8); RUN_STORE(2, 8); RUN_STORE(3, 8); RUN_STORE(5, 8); }
    else { RUN_STORE(0, 148); RUN_STORE(4, 148); RUN_STORE(1, 148); RUN_STORE(2, 148); RUN_STORE(3, 148); RUN_STORE(5, 148); }
  }
  fflush(stdout);

  CK(cudaFuncSetAttribute(mma_bench, cudaFuncAttributeMaxDynamicSharedMemorySize, SM));
  const int shapes[][2] = {{128, 256}, {128, 128}, {128, 64}, {128, 32}, {128, 16}, {64, 256}, {64, 128}, {64, 64}, {64, 32}};
  for (int g : {1, 148}) {
    for (auto& s : shapes) {
      mma_bench<<<g, 128, SM>>>(s[0], s[1], 256, cyc, err); CK(cudaDeviceSynchronize());
      const int iters = 4096;
      mma_bench<<<g, 128, SM>>>(s[0], s[1], iters, cyc, err); CK(cudaDeviceSynchronize());
      int herr = 0; CK(cudaMemcpy(&herr, err, 4, cudaMemcpyDeviceToHost));
      const double c = mean_cyc(cyc, g) / iters;
      printf("mma M=%3d N=%3d K=32 grid %3d: %.1f cycles/MMA  (%.0f MAC/clk/SM) err=%d\n", s[0], s[1], g, c, (double)s[0] * s[1] * 32 / c, herr);
    }
  }
  fflush(stdout);

  CK(cudaFuncSetAttribute(tld_bench<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, SM));
  CK(cudaFuncSetAttribute(tld_bench<32>, cudaFuncAttributeMaxDynamicSharedMemorySize, SM));
  for (int nw : {1, 4, 8}) {
    tld_bench<64><<<148, 384, SM>>>(nw, 2000, cyc, sink); CK(cudaDeviceSynchronize());
    printf("tcgen05.ld x64, %d warps active: %.1f cycles per ld+wait per warp\n", nw, mean_cyc(cyc, 8) / 2000);
    tld_bench<32><<<148, 384, SM>>>(nw, 2000, cyc, sink); CK(cudaDeviceSynchronize());
    printf("tcgen05.ld x32, %d warps active: %.1f cycles per ld+wait per warp\n", nw, mean_cyc(cyc, 8) / 2000);
  }
  fflush(stdout);

  CK(cudaFuncSetAttribute(bulk_bench, cudaFuncAttributeMaxDynamicSharedMemorySize, SM));
  for (int g : {8, 148}) for (int bytes : {128, 256, 512, 2048}) for (int lanes : {1, 32}) {
    const int iters = 512;
    bulk_bench<<<g, 128, SM>>>(buf, nrows, bytes, iters, lanes, cyc); CK(cudaDeviceSynchronize());
    const double c = mean_cyc(cyc, g);
    printf("bulk smem->global %4d B, %2d lanes, grid %3d: %.1f cycles per copy (issue lane), %.1f B/clk/SM\n", bytes, lanes, g, c / iters,
           (double)bytes * lanes * iters / c);
  }
  printf("done\n");
  return 0;
}
