// Record grouping helpers that mirror scannet/primitive_csr.py:23-29 (group_records: stable sort of
// record ids by primitive + bincount + cumsum) and scannet/primitive_gemm.py:186-203
// (prepare_groups: fixed-size segments of every primitive's record range).
//
// group_records is a device-wide stable LSD radix sort (4-bit digits) of (primitive id, record
// index) pairs.  A block owns 2048 consecutive items; inside it, chunks of 32 items are ranked with
// match.any, per-(digit, chunk) counts are scanned digit-major, and a global scan of per-block digit
// totals (digit-major, block-minor) gives every block its scatter bases, so equal ids keep their
// record order.
#include "frame.cuh"

namespace mlpsp {

int launch_scan_i32(const int32_t* in, int64_t n, int32_t* blk, int32_t* out, cudaStream_t st);

constexpr int kGsItems = 2048, kGsThreads = 256, kGsChunks = kGsItems / 32;

__global__ void __launch_bounds__(kGsThreads) k_gs_hist(const uint32_t* __restrict__ keys, int64_t n, int shift,
                                                        int nblocks, int32_t* __restrict__ ghist) {
  __shared__ int h[16];
  if (threadIdx.x < 16) h[threadIdx.x] = 0;
  __syncthreads();
  const int64_t base = (int64_t)blockIdx.x * kGsItems;
  for (int j = threadIdx.x; j < kGsItems; j += kGsThreads)
    if (base + j < n) atomicAdd(&h[(keys[base + j] >> shift) & 15u], 1);
  __syncthreads();
  if (threadIdx.x < 16) ghist[threadIdx.x * nblocks + blockIdx.x] = h[threadIdx.x];
}

__global__ void __launch_bounds__(kGsThreads) k_gs_scatter(
    const uint32_t* __restrict__ keys, const uint32_t* __restrict__ vals, int64_t n, int shift, int nblocks,
    const int32_t* __restrict__ gbase, uint32_t* __restrict__ keys_out, uint32_t* __restrict__ vals_out) {
  __shared__ int cnt[16 * kGsChunks];
  __shared__ int warp_sums[32];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int64_t base = (int64_t)blockIdx.x * kGsItems;
  for (int i = tid; i < 16 * kGsChunks; i += kGsThreads) cnt[i] = 0;
  __syncthreads();
  for (int c = warp; c < kGsChunks; c += kGsThreads / 32) {
    const int64_t i = base + c * 32 + lane;
    const bool valid = i < n;
    const uint32_t d = valid ? ((keys[i] >> shift) & 15u) : 0xffffffffu;
    const uint32_t peers = __match_any_sync(0xffffffffu, d);
    if (valid && lane == __ffs(peers) - 1) cnt[d * kGsChunks + c] = __popc(peers);
  }
  __syncthreads();
  constexpr int per = 16 * kGsChunks / kGsThreads;  // 4
  int local = 0;
#pragma unroll
  for (int j = 0; j < per; ++j) local += cnt[tid * per + j];
  int total;
  int ex = block_exclusive_scan(local, warp_sums, total);
#pragma unroll
  for (int j = 0; j < per; ++j) { const int v = cnt[tid * per + j]; cnt[tid * per + j] = ex; ex += v; }
  __syncthreads();
  for (int c = warp; c < kGsChunks; c += kGsThreads / 32) {
    const int64_t i = base + c * 32 + lane;
    const bool valid = i < n;
    const uint32_t k = valid ? keys[i] : 0u;
    const uint32_t d = valid ? ((k >> shift) & 15u) : 0xffffffffu;
    const uint32_t peers = __match_any_sync(0xffffffffu, d);
    if (valid) {
      const int64_t dst = (int64_t)gbase[d * nblocks + blockIdx.x] + (cnt[d * kGsChunks + c] - cnt[d * kGsChunks]) +
                          __popc(peers & ((1u << lane) - 1u));
      keys_out[dst] = k;
      vals_out[dst] = vals[i];
    }
  }
}

__global__ void k_gs_init(const int32_t* __restrict__ ids, int64_t n, int nprim, uint32_t* __restrict__ keys,
                          uint32_t* __restrict__ vals, int32_t* __restrict__ counts) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int32_t p = ids[i];
  keys[i] = (uint32_t)p;
  vals[i] = (uint32_t)i;
  if (p >= 0 && p < nprim) atomicAdd(counts + p, 1);
}

__global__ void k_gs_finish(const uint32_t* __restrict__ vals, int64_t n, int64_t* __restrict__ order,
                            const int32_t* __restrict__ off32, int nprim, int64_t* __restrict__ offsets) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) order[i] = (int64_t)vals[i];
  if (i <= nprim) offsets[i] = (int64_t)off32[i];
}

// total64 (zeroed by the caller) receives the exact number of groups: the per-primitive counts and their
// prefix are 32-bit, and the host rejects a layout whose total does not fit
__global__ void k_groups_count(const int64_t* __restrict__ offsets, int n, int64_t seg, int32_t* __restrict__ cnt,
                               unsigned long long* __restrict__ total64) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  long long c = 0;
  if (i < n) {
    c = (offsets[i + 1] - offsets[i] + seg - 1) / seg;
    if (c < 0) c = 0;
    cnt[i] = (int32_t)(c > 2147483647LL ? 2147483647LL : c);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) c += __shfl_xor_sync(0xffffffffu, c, o);
  if ((threadIdx.x & 31) == 0 && c > 0) atomicAdd(total64, (unsigned long long)c);
}

__global__ void k_groups_fill(const int64_t* __restrict__ offsets, int n, int64_t seg, const int32_t* __restrict__ goff32,
                              int64_t* __restrict__ group_offsets, int64_t* __restrict__ primitives,
                              int64_t* __restrict__ starts, int64_t max_groups) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i > n) return;
  group_offsets[i] = goff32[i];
  if (i == n || !primitives || !starts) return;
  const int g0 = goff32[i], g1 = goff32[i + 1];
  for (int g = g0; g < g1; ++g)
    if (g < max_groups) { primitives[g] = i; starts[g] = offsets[i] + (int64_t)(g - g0) * seg; }
}

// scratch: counts[n+1] | off32[n+2] | scan blocks | ghist[16*nblocks] | gbase[16*nblocks+1] | 4 x uint32[R]
struct GsLayout { int64_t o[9]; int64_t bytes; };
static GsLayout gs_layout(int64_t R, int n) {
  GsLayout L;
  int64_t off = 0;
  auto take = [&](int64_t bytes) { int64_t o = off; off += align_up(bytes, 256); return o; };
  const int64_t nblocks = std::max<int64_t>((R + kGsItems - 1) / kGsItems, 1);
  L.o[0] = take(4 * ((int64_t)n + 1));
  L.o[1] = take(4 * ((int64_t)n + 2));
  const int64_t scan_n = std::max<int64_t>((int64_t)n + 1, 16 * nblocks);
  L.o[2] = take(4 * (scan_n / kScanItems + 4));
  L.o[3] = take(4 * 16 * nblocks);
  L.o[4] = take(4 * (16 * nblocks + 1));
  for (int i = 5; i < 9; ++i) L.o[i] = take(4 * R);
  L.bytes = off;
  return L;
}

}  // namespace mlpsp

using namespace mlpsp;

extern "C" int64_t mlpsp_group_records_scratch_bytes(int64_t num_records, int32_t n) {
  if (num_records < 0 || n < 0) return -1;
  return gs_layout(num_records, n).bytes;
}

extern "C" int mlpsp_group_records(const int32_t* primitive_ids, int64_t num_records, int32_t n, int64_t* offsets,
                                   int64_t* order, void* scratch, int64_t scratch_bytes, void* stream) {
  cudaStream_t st = (cudaStream_t)stream;
  MLPSP_REQUIRE(num_records >= 0 && n >= 0 && offsets, MLPSP_E_ARG, "mlpsp_group_records: bad arguments");
  MLPSP_REQUIRE(num_records < (1ll << 31), MLPSP_E_LIMIT, "mlpsp_group_records: more than 2^31-1 records");
  MLPSP_REQUIRE(num_records == 0 || (primitive_ids && order), MLPSP_E_ARG, "mlpsp_group_records: null pointer");
  const int64_t R = num_records;
  const int nblocks = (int)((R + kGsItems - 1) / kGsItems);
  GsLayout L = gs_layout(R, n);
  MLPSP_REQUIRE(scratch && scratch_bytes >= L.bytes, MLPSP_E_SCRATCH, "mlpsp_group_records: scratch needs %lld bytes",
                (long long)L.bytes);
  const int64_t o_cnt = L.o[0], o_off = L.o[1], o_blk = L.o[2], o_gh = L.o[3], o_gb = L.o[4];
  const int64_t o_k0 = L.o[5], o_k1 = L.o[6], o_v0 = L.o[7], o_v1 = L.o[8];
  char* b = (char*)scratch;
  int32_t* counts = (int32_t*)(b + o_cnt); int32_t* off32 = (int32_t*)(b + o_off); int32_t* blk = (int32_t*)(b + o_blk);
  int32_t* ghist = (int32_t*)(b + o_gh); int32_t* gbase = (int32_t*)(b + o_gb);
  uint32_t* k[2] = {(uint32_t*)(b + o_k0), (uint32_t*)(b + o_k1)};
  uint32_t* v[2] = {(uint32_t*)(b + o_v0), (uint32_t*)(b + o_v1)};
  MLPSP_CUDA_OK(cudaMemsetAsync(counts, 0, 4 * ((size_t)n + 1), st));
  if (R > 0) k_gs_init<<<(unsigned)((R + 255) / 256), 256, 0, st>>>(primitive_ids, R, n, k[0], v[0], counts);
  int rc = launch_scan_i32(counts, (int64_t)n, blk, off32, st);
  if (rc) return rc;
  if (n == 0) MLPSP_CUDA_OK(cudaMemsetAsync(off32, 0, 4, st));
  int cur = 0;
  int bits = 1;
  while (bits < 32 && (1ll << bits) < (int64_t)std::max(n, 1)) ++bits;
  for (int shift = 0; shift < bits && R > 0; shift += 4) {
    k_gs_hist<<<nblocks, kGsThreads, 0, st>>>(k[cur], R, shift, nblocks, ghist);
    rc = launch_scan_i32(ghist, 16ll * nblocks, blk, gbase, st);
    if (rc) return rc;
    k_gs_scatter<<<nblocks, kGsThreads, 0, st>>>(k[cur], v[cur], R, shift, nblocks, gbase, k[cur ^ 1], v[cur ^ 1]);
    cur ^= 1;
  }
  const int64_t span = std::max<int64_t>(R, (int64_t)n + 1);
  k_gs_finish<<<(unsigned)((span + 255) / 256), 256, 0, st>>>(v[cur], R, order, off32, n, offsets);
  return cuda_check(cudaGetLastError(), "group_records");
}

extern "C" int mlpsp_prepare_groups(const int64_t* offsets, int32_t n, int64_t segment_size, int64_t* group_offsets,
                                    int64_t* primitives, int64_t* starts, int64_t max_groups,
                                    int64_t* num_groups_host, void* stream) {
  cudaStream_t st = (cudaStream_t)stream;
  MLPSP_REQUIRE(offsets && group_offsets && n >= 0, MLPSP_E_ARG, "mlpsp_prepare_groups: null pointer");
  MLPSP_REQUIRE(segment_size > 0, MLPSP_E_ARG, "segment_size must be a positive integer");
  // three small work arrays in one allocation: counts | prefix | scan blocks | 64-bit total
  const size_t bytes = (size_t)align_up(4 * ((int64_t)n + 2), 256);
  const size_t blk_bytes = (size_t)align_up(4 * ((int64_t)n / kScanItems + 4), 256);
  char* work = nullptr;
  MLPSP_CUDA_OK(cudaMallocAsync(&work, 2 * bytes + blk_bytes + 256, st));
  int32_t* cnt = reinterpret_cast<int32_t*>(work);
  int32_t* goff = reinterpret_cast<int32_t*>(work + bytes);
  int32_t* blk = reinterpret_cast<int32_t*>(work + 2 * bytes);
  unsigned long long* total64 = reinterpret_cast<unsigned long long*>(work + 2 * bytes + blk_bytes);
  int32_t G = 0;
  unsigned long long total = 0;
  // the allocation is released on every path; the first error wins
  int rc = cuda_check(cudaMemsetAsync(goff, 0, bytes + blk_bytes + 256, st), "prepare_groups");
  if (!rc && n > 0) k_groups_count<<<(n + 255) / 256, 256, 0, st>>>(offsets, n, segment_size, cnt, total64);
  if (!rc) rc = launch_scan_i32(cnt, n, blk, goff, st);
  if (!rc) {
    k_groups_fill<<<(n + 256) / 256, 256, 0, st>>>(offsets, n, segment_size, goff, group_offsets, primitives, starts, max_groups);
    rc = cuda_check(cudaMemcpyAsync(&G, goff + n, 4, cudaMemcpyDeviceToHost, st), "prepare_groups");
  }
  if (!rc) rc = cuda_check(cudaMemcpyAsync(&total, total64, 8, cudaMemcpyDeviceToHost, st), "prepare_groups");
  if (!rc) rc = cuda_check(cudaStreamSynchronize(st), "prepare_groups");
  cudaFreeAsync(work, st);
  if (rc) return rc;
  MLPSP_REQUIRE(total <= 2147483647ull, MLPSP_E_LIMIT,
                "mlpsp_prepare_groups: %llu groups exceed the 32-bit group index (raise segment_size)", total);
  if (num_groups_host) *num_groups_host = G;
  return cuda_check(cudaGetLastError(), "prepare_groups");
}

// ------------------------------------------------------------------------------------------
// prepare_groups for callers that must not allocate.
//
// mlpsp_prepare_groups above takes its three small work arrays from cudaMallocAsync.  Some hosts of
// this library cannot do that: a renderer plugin whose embedding engine owns all device memory and
// forbids driver allocations after start-up, or a frame loop that must not hit the implicit device
// synchronisation and the latency of cudaMalloc/cudaFree.  For them the same computation runs on a
// fixed scratch area that is part of the library image: a file-scope __device__ array, present on
// every GPU that loads the library until the process exits (about 4 MiB).
//
// The array's name is only a host-side handle in host code, not a device address, so the device
// address is looked up once per device with cudaGetSymbolAddress (with that device current) and
// cached; kernels receive that pointer.  The first call on a device performs this look-up, so make
// that first call outside any stream capture.  All calls share the one array and it keeps the
// previous call's contents: the part that must start at zero is cleared on every call, and two
// calls that overlap on the GPU (different streams or threads) would race on it, so serialise them.
namespace mlpsp {

constexpr int kStaticGroupsMaxPrims = MLPSP_STATIC_GROUPS_MAX_PRIMITIVES;
constexpr int64_t kSgCntBytes = (4ll * (kStaticGroupsMaxPrims + 2) + 255) / 256 * 256;
constexpr int64_t kSgBlkBytes = (4ll * (kStaticGroupsMaxPrims / kScanItems + 4) + 255) / 256 * 256;
constexpr int64_t kSgBytes = 2 * kSgCntBytes + kSgBlkBytes + 256;   // counts | prefix | scan blocks | 64-bit total

static __device__ __align__(256) unsigned char g_static_groups_scratch[kSgBytes];
static void* g_static_groups_ptr[64] = {nullptr};   // device address of the array, per device ordinal

static int static_groups_scratch(char** out) {
  int dev = -1;
  MLPSP_CUDA_OK(cudaGetDevice(&dev));
  MLPSP_REQUIRE(dev >= 0 && dev < 64, MLPSP_E_LIMIT, "mlpsp_prepare_groups_static: device ordinal %d beyond 63", dev);
  if (!g_static_groups_ptr[dev]) {
    void* p = nullptr;
    MLPSP_CUDA_OK(cudaGetSymbolAddress(&p, g_static_groups_scratch));
    MLPSP_REQUIRE(p != nullptr, MLPSP_E_CUDA, "mlpsp_prepare_groups_static: no device address for the scratch array");
    g_static_groups_ptr[dev] = p;
  }
  *out = static_cast<char*>(g_static_groups_ptr[dev]);
  return MLPSP_OK;
}

}  // namespace mlpsp

extern "C" int mlpsp_prepare_groups_static(const int64_t* offsets, int32_t n, int64_t segment_size,
                                           int64_t* group_offsets, int64_t* primitives, int64_t* starts,
                                           int64_t max_groups, int64_t* num_groups_host, void* stream) {
  cudaStream_t st = (cudaStream_t)stream;
  MLPSP_REQUIRE(offsets && group_offsets && n >= 0, MLPSP_E_ARG, "mlpsp_prepare_groups_static: null pointer");
  MLPSP_REQUIRE(segment_size > 0, MLPSP_E_ARG, "segment_size must be a positive integer");
  MLPSP_REQUIRE(n <= kStaticGroupsMaxPrims, MLPSP_E_LIMIT,
                "mlpsp_prepare_groups_static: %d primitives exceed the built-in scratch capacity of %d "
                "(MLPSP_STATIC_GROUPS_MAX_PRIMITIVES); use mlpsp_prepare_groups", n, kStaticGroupsMaxPrims);
  char* base = nullptr;
  int rc = static_groups_scratch(&base);
  if (rc) return rc;
  int32_t* cnt = reinterpret_cast<int32_t*>(base);
  int32_t* goff = reinterpret_cast<int32_t*>(base + kSgCntBytes);
  int32_t* blk = reinterpret_cast<int32_t*>(base + 2 * kSgCntBytes);
  unsigned long long* total64 = reinterpret_cast<unsigned long long*>(base + 2 * kSgCntBytes + kSgBlkBytes);
  // the prefix array must read zero where the scan does not write (n == 0) and must not show the
  // previous call's totals; the 64-bit group total starts at zero as well
  MLPSP_CUDA_OK(cudaMemsetAsync(goff, 0, 4 * ((size_t)n + 2), st));
  MLPSP_CUDA_OK(cudaMemsetAsync(total64, 0, 8, st));
  if (n > 0) k_groups_count<<<(n + 255) / 256, 256, 0, st>>>(offsets, n, segment_size, cnt, total64);
  rc = launch_scan_i32(cnt, n, blk, goff, st);
  if (rc) return rc;
  k_groups_fill<<<(n + 256) / 256, 256, 0, st>>>(offsets, n, segment_size, goff, group_offsets, primitives, starts, max_groups);
  int32_t G = 0;
  unsigned long long total = 0;
  MLPSP_CUDA_OK(cudaMemcpyAsync(&G, goff + n, 4, cudaMemcpyDeviceToHost, st));
  MLPSP_CUDA_OK(cudaMemcpyAsync(&total, total64, 8, cudaMemcpyDeviceToHost, st));
  MLPSP_CUDA_OK(cudaStreamSynchronize(st));
  MLPSP_REQUIRE(total <= 2147483647ull, MLPSP_E_LIMIT,
                "mlpsp_prepare_groups_static: %llu groups exceed the 32-bit group index (raise segment_size)", total);
  if (num_groups_host) *num_groups_host = G;
  return cuda_check(cudaGetLastError(), "prepare_groups_static");
}
