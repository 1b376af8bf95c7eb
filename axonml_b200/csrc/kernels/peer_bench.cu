// Micro-benchmarks of the peer-memory paths the fused collectives use: stores to a peer (bulk
// stores from shared memory, or per-thread 16-byte stores) and loads of peer-written symmetric
// memory in several flavours.  No kernel here waits on another rank; they only move bytes.
// Driver: python -m axonml_b200.parallel.bench_peer_copy
#include "common.cuh"

namespace {
using namespace ax;

// mode 0: lane 0 of every warp runs a pipeline of `piece`-byte bulk stores, `depth` pieces of
//         shared memory per CTA;  mode 1: every thread issues 16-byte stores
__global__ void __launch_bounds__(512, 1)
peer_store_kernel(uint8_t* __restrict__ dst_base, long bytes_per_cta, int piece, int depth, int mode) {
  extern __shared__ __align__(128) uint8_t psmem[];
  uint8_t* dst = dst_base + (long)blockIdx.x * bytes_per_cta;
  if (mode == 0) {
    for (int i = threadIdx.x; i < piece * depth / 16; i += blockDim.x) ((uint4*)psmem)[i] = make_uint4(i, 1, 2, 3);
    fence_proxy_async_smem();
    __syncthreads();
    const int warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    if ((threadIdx.x & 31) == 0) {
      const long per_w = bytes_per_cta / nw;
      uint8_t* d = dst + warp * per_w;
      const int my_depth = depth / nw > 0 ? depth / nw : 1;
      uint8_t* sb = psmem + (long)warp * my_depth * piece;
      const long n = per_w / piece;
      for (long i = 0; i < n; ++i) {
        asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(d + i * piece),
                     "r"(smem_u32(sb + (i % my_depth) * piece)), "r"(piece)
                     : "memory");
        tma_store_commit();
        if (my_depth >= 8) tma_store_wait_read<7>();
        else if (my_depth >= 4) tma_store_wait_read<3>();
        else if (my_depth >= 2) tma_store_wait_read<1>();
        else tma_store_wait_read<0>();
      }
      tma_store_wait<0>();
    }
  } else {
    const long n16 = bytes_per_cta / 16;
    const uint4 v = make_uint4(threadIdx.x, 1, 2, 3);
    for (long i = threadIdx.x; i < n16; i += blockDim.x)
      asm volatile("st.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(dst + i * 16), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
  }
}

template <int MODE>
__device__ __forceinline__ uint4 load_flavour(const void* p) {
  uint4 v;
  if (MODE == 0) asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  if (MODE == 1) asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  if (MODE == 2) asm volatile("ld.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  if (MODE == 3) asm volatile("ld.relaxed.gpu.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}

// every warp reads 4 KB pieces the way the reduce-scatter epilogue does (lane = one 128-byte row)
template <int MODE>
__global__ void __launch_bounds__(128, 1)
peer_load_kernel(const uint8_t* __restrict__ src, long bytes_per_cta, unsigned* sink, unsigned long long* ns) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint8_t* base = src + (long)blockIdx.x * bytes_per_cta + (long)warp * (bytes_per_cta / 4);
  const long pieces = bytes_per_cta / 4 / 4096;
  unsigned acc = 0;
  const unsigned long long t0 = globaltimer_ns();
  for (long i = 0; i < pieces; ++i) {
    const uint8_t* p = base + i * 4096 + lane * 128;
    uint4 u[8];
#pragma unroll
    for (int c = 0; c < 8; ++c) u[c] = load_flavour<MODE>(p + ((c ^ (lane & 7)) << 4));
#pragma unroll
    for (int c = 0; c < 8; ++c) acc += u[c].x ^ u[c].y ^ u[c].z ^ u[c].w;
  }
  const unsigned long long t1 = globaltimer_ns();
  if (acc == 0x12345678u) sink[0] = acc;
  if (threadIdx.x == 0) ns[blockIdx.x] = t1 - t0;
}

}  // namespace

AX_API int ax_peer_store_bench(void* dst, long bytes_per_cta, int piece, int depth, int mode, int grid, int threads,
                               cudaStream_t stream) {
  if (grid < 1 || threads < 32 || threads > 512 || threads % 32) return -1;
  if (mode == 0 && (piece % 16 || piece * depth > 200 * 1024 || bytes_per_cta % ((long)piece * (threads / 32)))) return -1;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(peer_store_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  peer_store_kernel<<<grid, threads, mode == 0 ? piece * depth : 0, stream>>>((uint8_t*)dst, bytes_per_cta, piece, depth, mode);
  return (int)cudaGetLastError();
}

AX_API int ax_peer_load_bench(int flavour, const void* src, long bytes_per_cta, void* sink, void* ns, int grid,
                              cudaStream_t stream) {
  if (grid < 1 || bytes_per_cta % (4 * 4096)) return -1;
  auto* s = (const uint8_t*)src;
  auto* k = (unsigned*)sink;
  auto* t = (unsigned long long*)ns;
  switch (flavour) {
    case 0: peer_load_kernel<0><<<grid, 128, 0, stream>>>(s, bytes_per_cta, k, t); break;
    case 1: peer_load_kernel<1><<<grid, 128, 0, stream>>>(s, bytes_per_cta, k, t); break;
    case 2: peer_load_kernel<2><<<grid, 128, 0, stream>>>(s, bytes_per_cta, k, t); break;
    case 3: peer_load_kernel<3><<<grid, 128, 0, stream>>>(s, bytes_per_cta, k, t); break;
    default: return -1;
  }
  return (int)cudaGetLastError();
}
