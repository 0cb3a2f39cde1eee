// Per-primitive MLP evaluator on the 5th-generation tensor cores (tcgen05, sm_100a).
//
// What the reference does per (tile, primitive) with warp-level wmma on 64 rays
// (scannet/cuda/rgb_wmma.cuh:75-223) is done here per (primitive, 128 of its records):
//   * the primitive's weight image (packed once per scene in the canonical K-major core-matrix
//     layout, biases included) arrives in shared memory in three pieces, one per layer, each by a TMA
//     bulk copy (cp.async.bulk) that signals its own mbarrier;
//   * each of the 128 worker threads owns one record (row): it encodes the record (sin / cos of 36 phases),
//     rounds to the operand format and stores straight into the K-major A tile;
//   * layer 1 (128x80 . 80xH), layer 2 (128xH . HxH) and layer 3 (128xH . Hx16, 4 columns used) are
//     tcgen05.mma.kind::f16 instructions issued by one lane of a fifth warp, FP32 accumulators in tensor memory.
//     The biases ride in the same instructions: one extra K step per layer multiplies a constant row
//     of ones (eight rows of shared memory, broadcast to all 128 by a zero row stride) with the bias
//     split into up to eight operand-format terms, so no thread ever adds a bias;
//   * between layers every thread pulls its accumulator row back with tcgen05.ld, applies ReLU while
//     rounding to the operand format and writes the next A tile; the epilogue applies sigmoid /
//     softplus (and 1-exp(-sigma*decay)) and scatters one float4 per record to its compositing slot.
// The three layers of item i, the encoding of item i+1 and the output of item i-1 are software-pipelined:
// every wait for a group of MMAs is preceded by independent work of a neighbouring item, so the
// special-function pipe (the binding unit of this kernel) stays busy while the tensor pipe turns around.
//
// Numerics follow the reference's tensor-core contract: operands and hidden activations rounded
// to binary16 / bfloat16 (RN), FP32 accumulation from zero.
//
// Every wait on an mbarrier is bounded; when one gives up the CTA raises MLPSP_ST_TIMEOUT, waits
// (bounded) for its own copies, frees its tensor memory and returns.
#include "frame.cuh"
#include "tc.cuh"

namespace mlpsp {

constexpr int kRows = kRowsPerItem;      // 128 = MMA M
constexpr int kChunk = kRows * 16;       // bytes of one K chunk of an A tile: [128 rows][8 halves]
constexpr int kN3 = 16;                  // 4 outputs padded to the smallest N
constexpr int kA1Chunks = 9;             // 72 encoded inputs

// ---- packed weight image (per primitive) and shared-memory plan for F = 6, hidden width H = 32 or 64 ----
// piece 1: W1 as [11 chunks][H rows][8 halves]: chunks 0..8 hold K = 0..71 in the order of enc_k(), chunk 9 is
//          zero (it meets whatever follows the last A chunk), chunk 10 holds the eight terms of b1[h];
// piece 2: W2 as [H/8 + 1 chunks][H][8], the last one the terms of b2;
// piece 3: W3 as [H/8 + 1 chunks][16][8] (rows 4..15 zero), the last one the terms of b3.
template <int H>
struct Net {
  static_assert(H == 32 || H == 64, "hidden width of the tensor-core evaluator");
  static constexpr int kWChunk = H * 16;
  static constexpr int kW3Chunk = kN3 * 16;
  static constexpr int kOffW1 = 0;
  static constexpr int kBytesW1 = 11 * kWChunk;
  static constexpr int kOffW2 = kOffW1 + kBytesW1;
  static constexpr int kBytesW2 = (H / 8 + 1) * kWChunk;
  static constexpr int kOffW3 = kOffW2 + kBytesW2;
  static constexpr int kBytesW3 = (H / 8 + 1) * kW3Chunk;
  static constexpr int kWeightBytes = kOffW3 + kBytesW3;          // 9,472 (H = 32) / 22,784 (H = 64)
  // shared memory: weight image | eight rows of ones, eight rows of zeros | layer-1 A tile | hidden A tile | barriers.
  // The order matters: the second chunk of a bias K step on the weight side is "whatever follows" (the next
  // piece, or the ones / zeros after the image), always finite, and meets the zero rows on the A side; the second
  // chunk of the last layer-1 K step on the A side is the first hidden chunk and meets W1's zero chunk.
  static constexpr int kOffConst = kWeightBytes;
  static constexpr int kOffA1 = kOffConst + 256;
  static constexpr int kOffA2 = kOffA1 + kA1Chunks * kChunk;
  static constexpr int kOffBar = kOffA2 + (H / 8) * kChunk;
  static constexpr int kSmemBytes = kOffBar + 96;                  // 36,448 / 57,952
  static constexpr int kTmemCols = 2 * H;   // D1 [0,H)  D2 [H,2H)  D3 [H,H+16)
  // resident CTAs per SM: H = 32: shared memory would give 6, five leave each thread 80 registers (no spills; six
  // measured no faster); H = 64: shared memory gives 3
  static constexpr int kCtas = H == 32 ? 5 : 3;
  static_assert(kWeightBytes % 16 == 0 && kBytesW1 % 16 == 0 && kBytesW2 % 16 == 0 && kBytesW3 % 16 == 0, "bulk-copy granularity");
};

// Position of an encoded input inside the K dimension of layer 1.  The reference orders K as
// [sin(c,f) for c, f][cos(c,f) for c, f] (np_tile_kernels.cu:329-343); a dot product does not care, so
// the A tile and the packed W1 rows both use an order in which the six (sin, cos) pairs of one input
// coordinate are contiguous (six 32-bit words per coordinate):
//   k' = 12 c + 4 (f / 2) + 2 is_cos + (f % 2).
__host__ __device__ constexpr int enc_k(int c, int f, int is_cos) { return 12 * c + 4 * (f >> 1) + 2 * is_cos + (f & 1); }
__host__ __device__ constexpr int enc_k_of_reference(int k) {
  return k >= 72 ? k : enc_k((k % 36) / 6, (k % 36) % 6, k / 36);
}

// The six words of one input coordinate.  mult[f] is freq[f] * att[f].  LADDER: every band is exactly twice the
// one before, so the phases are exact doublings of the first and sin / cos of the higher bands follow from the
// double-angle identities (2 special-function evaluations per coordinate instead of 12).
template <bool LADDER, bool BF16>
__device__ __forceinline__ void encode_coord(float v, const float (&mult)[6], uint32_t (&w)[6]) {
  float sn[6], cs[6];
  if (LADDER) {
    __sincosf(v * mult[0], &sn[0], &cs[0]);
#pragma unroll
    for (int f = 1; f < 6; ++f) {
      const float t = sn[f - 1] + sn[f - 1];
      sn[f] = t * cs[f - 1];
      cs[f] = fmaf(-t, sn[f - 1], 1.0f);
    }
  } else {
#pragma unroll
    for (int f = 0; f < 6; ++f) __sincosf(v * mult[f], &sn[f], &cs[f]);
  }
#pragma unroll
  for (int g = 0; g < 3; ++g) {
    w[g * 2] = pack_h2<BF16>(sn[2 * g], sn[2 * g + 1]);
    w[g * 2 + 1] = pack_h2<BF16>(cs[2 * g], cs[2 * g + 1]);
  }
}

// a finite input gives finite phases (freq * att <= 101)
__device__ __forceinline__ bool not_finite(float v) { return !(fabsf(v) < 1.0e30f); }

// The first and the second part of a record's encoding, written to this thread's row of the layer-1 A tile
// (row = generic pointer to the row's 16 bytes inside chunk 0; kChunk = bytes between the K chunks of the tile).
// q0 = (rdx, rdy, rdz, dx), q1 = (dy, dz, decay, slot) are the record's two 16-byte halves; part 1 computes
// coordinates 0..3 (chunks 0..5), part 2 coordinates 4 and 5.
template <bool LADDER, bool BF16, int kChunk = mlpsp::kChunk>
__device__ __forceinline__ bool encode_part1(const float4 q0, const float (&mult)[6], char* row) {
  uint32_t a[6], b[6];
  encode_coord<LADDER, BF16>(q0.x, mult, a);
  encode_coord<LADDER, BF16>(q0.y, mult, b);
  *reinterpret_cast<uint4*>(row) = make_uint4(a[0], a[1], a[2], a[3]);
  *reinterpret_cast<uint4*>(row + kChunk) = make_uint4(a[4], a[5], b[0], b[1]);
  *reinterpret_cast<uint4*>(row + 2 * kChunk) = make_uint4(b[2], b[3], b[4], b[5]);
  encode_coord<LADDER, BF16>(q0.z, mult, a);
  encode_coord<LADDER, BF16>(q0.w, mult, b);
  *reinterpret_cast<uint4*>(row + 3 * kChunk) = make_uint4(a[0], a[1], a[2], a[3]);
  *reinterpret_cast<uint4*>(row + 4 * kChunk) = make_uint4(a[4], a[5], b[0], b[1]);
  *reinterpret_cast<uint4*>(row + 5 * kChunk) = make_uint4(b[2], b[3], b[4], b[5]);
  return not_finite(q0.x) || not_finite(q0.y) || not_finite(q0.z) || not_finite(q0.w);
}
template <bool LADDER, bool BF16, int kChunk = mlpsp::kChunk>
__device__ __forceinline__ bool encode_part2(const float4 q1, const float (&mult)[6], char* row) {
  uint32_t a[6], b[6];
  encode_coord<LADDER, BF16>(q1.x, mult, a);
  encode_coord<LADDER, BF16>(q1.y, mult, b);
  *reinterpret_cast<uint4*>(row + 6 * kChunk) = make_uint4(a[0], a[1], a[2], a[3]);
  *reinterpret_cast<uint4*>(row + 7 * kChunk) = make_uint4(a[4], a[5], b[0], b[1]);
  *reinterpret_cast<uint4*>(row + 8 * kChunk) = make_uint4(b[2], b[3], b[4], b[5]);
  return not_finite(q1.x) || not_finite(q1.y);
}

// hidden layer epilogue: ReLU, operand format (RN), write this thread's row of the hidden A tile.  The biases are
// already in the accumulators.  Returns true when an activation rounded to +inf.  The FP32 sums themselves are
// finite for finite operands (rgb_wmma.cuh:179-181 checks for a non-finite or overflowing activation per element).
template <bool KEEP, bool BF16, int kChunk = mlpsp::kChunk>
__device__ __forceinline__ bool hidden_to_smem(const uint32_t (&acc)[32], char* a2, int row, uint32_t& relu_mask) {
  // running maximum of the packed activations (they are >= 0 after the ReLU, so for both formats the bit
  // patterns order like the values and one unsigned 16-bit-lane maximum serves either)
  uint32_t top = 0u;
  relu_mask = 0u;
#pragma unroll
  for (int kc = 0; kc < 4; ++kc) {
    uint32_t w[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const int j = kc * 8 + q * 2;
      const float v0 = __uint_as_float(acc[j]), v1 = __uint_as_float(acc[j + 1]);
      if (KEEP) {
        relu_mask |= (v0 > 0.f ? 1u : 0u) << j;
        relu_mask |= (v1 > 0.f ? 1u : 0u) << (j + 1);
      }
      w[q] = pack_h2_relu<BF16>(v0, v1);
      top = __vmaxu2(top, w[q]);
    }
    *reinterpret_cast<uint4*>(a2 + kc * kChunk + row * 16) = make_uint4(w[0], w[1], w[2], w[3]);
  }
  // +inf (or the canonical NaN a non-finite sum converts to) in either lane
  const uint32_t inf16 = BF16 ? 0x7f80u : 0x7c00u;
  return (top & 0xffffu) >= inf16 || (top >> 16) >= inf16;
}

// One work item = (primitive, first record, rows <= 128).  Items are dealt to CTAs round-robin
// (item = blockIdx.x + k * gridDim.x): all items cost about the same, and a fixed deal lets a CTA
// fetch the next items' descriptors, records and weight pieces while the current item is in flight.
//
// A CTA is four worker warps (one record per thread) and one issue warp.  Nothing in the steady state is a
// CTA-wide barrier: the workers tell the issue warp that an operand tile is complete through an mbarrier that
// counts one arrival per worker warp, the issue warp (one lane) waits for that and for the layer's weight piece,
// issues the layer's MMAs and commits them to the mbarrier the workers wait on.  It also refills each weight
// piece as soon as the MMAs that read it have finished.  A worker warp, item i ("|" = while the MMAs run):
//   layer-1 tile of i complete -> arrive | output of i-1 (its layer-3 MMAs have finished by now)
//   wait layer 1: hidden tile 1 of i written -> arrive | first part of the encoding of i+1
//   wait layer 2: hidden tile 2 of i written -> arrive | second part of the encoding of i+1
constexpr int kMlpThreads = kRows + 32;

template <bool KEEP, bool BF16, int H>
__global__ void __launch_bounds__(kMlpThreads, Net<H>::kCtas) k_mlp_tc(
    const char* __restrict__ w16, const float* __restrict__ freq, const float* __restrict__ att,
    const float4* __restrict__ rec_in, const int4* __restrict__ work,
    const int32_t* __restrict__ counters, float4* __restrict__ rec_out, float4* __restrict__ rec_ext, int out_mode,
    int32_t* __restrict__ status) {
  using N = Net<H>;
  static_assert(!KEEP || H == 32, "the record export keeps 32-bit ReLU masks");
  chain_wait();       // the work list and the records come from the previous kernels of the frame
  chain_release();
  extern __shared__ __align__(128) char smem[];
  char* s_a1 = smem + N::kOffA1;
  char* s_a2 = smem + N::kOffA2;
  // [0..2] weight pieces landed, [3..5] operand tile of layer 1 / 2 / 3 complete, [6] layer-1 MMAs done, [7] layer-2 / 3 MMAs done
  uint64_t* s_bar = reinterpret_cast<uint64_t*>(smem + N::kOffBar);
  uint32_t* s_misc = reinterpret_cast<uint32_t*>(s_bar + 8);          // [0] tmem base, [1] a wait gave up
  if (status[MLPSP_ST_BITS] & MLPSP_ST_FATAL) return;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int G = counters[kCtrWork];
  int item = blockIdx.x;
  if (item >= G) return;                     // more CTAs than work: leave before touching tensor memory
  const int stride = (int)gridDim.x;
  const uint32_t wb = smem_u32(smem), cst = wb + N::kOffConst, a1 = wb + N::kOffA1, a2 = wb + N::kOffA2;
  const uint32_t bar_w0 = smem_u32(&s_bar[0]), bar_r0 = smem_u32(&s_bar[3]), bar_a = smem_u32(&s_bar[6]), bar_b = smem_u32(&s_bar[7]);
  if (tid == 0) {
#pragma unroll
    for (int b = 0; b < 3; ++b) { mbar_init(bar_w0 + 8 * b, 1); mbar_init(bar_r0 + 8 * b, kRows / 32); }
    mbar_init(bar_a, 1);
    mbar_init(bar_b, 1);
    s_misc[1] = 0u;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == kRows / 32) tmem_alloc(smem_u32(&s_misc[0]), N::kTmemCols);
  // eight rows of ones, eight rows of zeros; the hidden tile starts finite (its first chunk is read, against zero
  // weights, by the first layer-1 MMAs before any activation has been written)
  if (tid < 16) {
    const uint32_t one2 = BF16 ? 0x3f803f80u : 0x3c003c00u;
    const uint32_t v = tid < 8 ? one2 : 0u;
    *reinterpret_cast<uint4*>(smem + N::kOffConst + tid * 16) = make_uint4(v, v, v, v);
  }
  if (tid < kRows) {
#pragma unroll
    for (int c = 0; c < H / 8; ++c) *reinterpret_cast<uint4*>(s_a2 + c * kChunk + tid * 16) = make_uint4(0u, 0u, 0u, 0u);
  }
  fence_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = s_misc[0];
  bool ok = true;

  if (warp == kRows / 32) {
    // ------------------------------------------------------------------ issue warp ----
    if (lane == 0) {
      const uint64_t ones_desc = smem_desc(cst, 128, 0);   // rows of ones, then rows of zeros; every row group the same
      const uint32_t idesc_h = instr_desc(kRows, H, BF16), idesc_o = instr_desc(kRows, kN3, BF16);
      // Operand descriptors are built once; a K step only moves the start address, which sits in the low bits in
      // units of 16 bytes (shared-memory addresses stay below 2^18, so the sum never carries out of the field).
      const uint64_t a1_desc = smem_desc(a1, kChunk, 128), a2_desc = smem_desc(a2, kChunk, 128);
      const uint64_t w1_desc = smem_desc(wb + N::kOffW1, N::kWChunk, 128), w2_desc = smem_desc(wb + N::kOffW2, N::kWChunk, 128);
      const uint64_t w3_desc = smem_desc(wb + N::kOffW3, N::kW3Chunk, 128);
      auto step = [](uint64_t desc, int bytes) { return desc + (uint64_t)(bytes >> 4); };
      auto request = [&](int piece, int prim) {
        const int off = piece == 0 ? N::kOffW1 : (piece == 1 ? N::kOffW2 : N::kOffW3);
        const int bytes = piece == 0 ? N::kBytesW1 : (piece == 1 ? N::kBytesW2 : N::kBytesW3);
        mbar_expect_tx(bar_w0 + 8 * piece, bytes);
        bulk_g2s(wb + off, w16 + (size_t)prim * N::kWeightBytes + off, bytes, bar_w0 + 8 * piece);
      };
      int prim = __ldg(work + item).x;
      uint32_t pend = 7u;                    // weight pieces requested and not yet waited for
      request(0, prim); request(1, prim); request(2, prim);
      uint32_t li = 0u;
      for (;;) {
        const uint32_t par = li & 1u;
        const int next = item + stride;
        const bool has_next = next < G;
        int prim_n = 0;
        if (has_next) prim_n = __ldg(work + next).x;
        // ---- layer 1: D1[128xH] = A1[128x72] . W1^T + b1 ----
        ok = mbar_wait(bar_r0, par) && mbar_wait(bar_w0, par);
        pend &= ~1u;
        // The second chunk of a bias K step reads the start of the next piece's region as don't-care data (it meets
        // zeros), which must still be finite: before the first item all three pieces have to be in place, afterwards
        // the regions always hold the previous or the incoming image.
        if (ok && li == 0u) { ok = mbar_wait(bar_w0 + 8, 0u) && mbar_wait(bar_w0 + 16, 0u); }
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int ks = 0; ks < 4; ++ks)
          mma_f16(tmem, step(a1_desc, ks * 2 * kChunk), step(w1_desc, ks * 2 * N::kWChunk), idesc_h, ks > 0);
        // K = 64..79: the last A chunk and whatever follows it (the first hidden chunk) meet W1's chunk 8 and zeros
        mma_f16(tmem, step(a1_desc, 8 * kChunk), step(w1_desc, 8 * N::kWChunk), idesc_h, 1u);
        mma_f16(tmem, ones_desc, step(w1_desc, 10 * N::kWChunk), idesc_h, 1u);
        mma_commit(bar_a);
        if (!mbar_wait(bar_a, par)) { ok = false; break; }
        if (has_next) { request(0, prim_n); pend |= 1u; }          // W1 is no longer read
        // ---- layer 2: D2[128xH] = H1[128xH] . W2^T + b2 ----
        ok = mbar_wait(bar_r0 + 8, par) && mbar_wait(bar_w0 + 8, par);
        pend &= ~2u;
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int ks = 0; ks < H / 16; ++ks)
          mma_f16(tmem + H, step(a2_desc, ks * 2 * kChunk), step(w2_desc, ks * 2 * N::kWChunk), idesc_h, ks > 0);
        mma_f16(tmem + H, ones_desc, step(w2_desc, (H / 8) * N::kWChunk), idesc_h, 1u);
        mma_commit(bar_b);
        if (!mbar_wait(bar_b, 0u)) { ok = false; break; }
        if (has_next) { request(1, prim_n); pend |= 2u; }
        // ---- layer 3: D3[128x16] = H2[128xH] . W3^T + b3 (rows 4..15 of W3 are zero) ----
        ok = mbar_wait(bar_r0 + 16, par) && mbar_wait(bar_w0 + 16, par);
        pend &= ~4u;
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int ks = 0; ks < H / 16; ++ks)
          mma_f16(tmem + H, step(a2_desc, ks * 2 * kChunk), step(w3_desc, ks * 2 * N::kW3Chunk), idesc_o, ks > 0);
        mma_f16(tmem + H, ones_desc, step(w3_desc, (H / 8) * N::kW3Chunk), idesc_o, 1u);
        mma_commit(bar_b);
        if (!mbar_wait(bar_b, 1u)) { ok = false; break; }
        if (!has_next) break;
        request(2, prim_n); pend |= 4u;
        item = next;
        prim = prim_n;
        ++li;
      }
      if (!ok) {
        s_misc[1] = 1u;
        // our own bulk copies may still be in flight: give them a bounded chance to land before the CTA's
        // shared memory is released
        for (int b = 0; b < 3; ++b)
          if (pend & (1u << b)) mbar_wait(bar_w0 + 8 * b, li & 1u);
      }
    }
    __syncwarp();
  } else {
    // ---------------------------------------------------------------- worker warps ----
    const uint32_t trow = tmem + ((uint32_t)(warp * 32) << 16);   // this warp's 32 lanes
    // phase multipliers freq[f] * att[f]; when every band is exactly twice the one before (equal
    // attenuation: FourierFeatureEncoding's bands, cumodel.py:163) the encoder takes the double-angle route
    float mult[6];
    bool ladder = true;
#pragma unroll
    for (int f = 0; f < 6; ++f) mult[f] = __ldg(freq + f) * __ldg(att + f);
#pragma unroll
    for (int f = 1; f < 6; ++f) ladder = ladder && mult[f] == 2.0f * mult[f - 1];
    int4 wk = __ldg(work + item);
    int4 wk_n = (item + stride < G) ? __ldg(work + item + stride) : make_int4(0, 0, 0, 0);
    auto load_rec = [&](const int4& w, float4& r0, float4& r1) {
      r0 = make_float4(0.f, 0.f, 0.f, 0.f);
      r1 = make_float4(0.f, 0.f, 0.f, 0.f);     // the zero record, never stored
      if (tid < w.z) { r0 = __ldg(rec_in + 2 * (size_t)(w.y + tid)); r1 = __ldg(rec_in + 2 * (size_t)(w.y + tid) + 1); }
    };
    auto rec_decay = [](const float4& r1) { return r1.z; };
    auto rec_slot = [](const float4& r1) { return __float_as_uint(r1.w); };
    // the warp's rows of an operand tile are complete (and its reads of tensor memory have retired)
    auto tile_done = [&](uint32_t bar) {
      fence_async_smem();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
    };
    char* my_row = s_a1 + tid * 16;
    bool bad = false;

    // ---- prologue: the first item's record, encoded in full ----
    float4 q0, q1;
    load_rec(wk, q0, q1);
    // MMA rows are independent and rows past the end of the primitive's records are never stored, so a
    // warp whose 32 rows are all past the end skips the encoding and the epilogues (its rows of the
    // operand tiles keep whatever they held) and only reports its tiles complete
    if (warp * 32 < wk.z) {
      // rows past the end inside a live warp hold the zero record; their results are never stored
      if (ladder) { bad |= encode_part1<true, BF16>(q0, mult, my_row); bad |= encode_part2<true, BF16>(q1, mult, my_row); }
      else { bad |= encode_part1<false, BF16>(q0, mult, my_row); bad |= encode_part2<false, BF16>(q1, mult, my_row); }
    }
    tile_done(bar_r0);
    float decay_c = rec_decay(q1);
    uint32_t slot_c = rec_slot(q1);
    load_rec(wk_n, q0, q1);                    // the second item's record (zero record when there is none)

    bool have_prev = false, live_p = false, valid_p = false;
    float decay_p = 0.f;
    uint32_t slot_p = 0u, relu1 = 0u, relu2 = 0u, relu1_p = 0u, relu2_p = 0u;
    uint32_t li = 0u;                          // items this CTA has started: parity of the once-per-item barriers

    auto emit_output = [&]() {
      // output of the item whose layer-3 MMAs have just finished: (decay_p, slot_p), accumulator columns [H, H+4)
      if (!live_p) return;
      uint32_t o[4];
      tmem_ld4(trow + H, o);
      if (valid_p) {
        const float o0 = __uint_as_float(o[0]), o1 = __uint_as_float(o[1]), o2 = __uint_as_float(o[2]), o3 = __uint_as_float(o[3]);
        const float sigma_raw = softplus_fast(o3);
        float4 out;
        out.x = sigmoid_fast(o0); out.y = sigmoid_fast(o1); out.z = sigmoid_fast(o2);
        out.w = (out_mode == kOutAlpha) ? (1.f - __expf(-(sigma_raw * decay_p))) : sigma_raw;
        rec_out[slot_p] = out;
        if (KEEP) rec_ext[slot_p] = make_float4(sigma_raw, o3, __uint_as_float(relu1_p), __uint_as_float(relu2_p));
      }
    };

    for (;;) {
      const int nrows = wk.z;
      const bool valid = tid < nrows;
      const bool warp_live = warp * 32 < nrows;
      const int next = item + stride;
      const bool has_next = next < G;
      const bool next_live = has_next && warp * 32 < wk_n.z;
      const uint32_t par = li & 1u;
      // descriptor of the item after the next one
      const int next2 = next + stride;
      int4 wk_n2 = make_int4(0, 0, 0, 0);
      if (next2 < G) wk_n2 = __ldg(work + next2);
      // ---- output of the previous item while layer 1 of this one runs ----
      if (have_prev) {
        ok = __all_sync(0xffffffffu, mbar_wait(bar_b, 1u) && ok);   // warp-uniform: tcgen05.ld is .sync.aligned
        tc_fence_after();
        if (!ok) break;
        emit_output();
      }
      ok = __all_sync(0xffffffffu, mbar_wait(bar_a, par) && ok);
      tc_fence_after();
      if (!ok) break;
      // the record this thread will load at the end of this item (for the item after the next) is asked into L2 now
      if (tid < wk_n2.z) asm volatile("prefetch.global.L2 [%0];" ::"l"(rec_in + 2 * (size_t)(wk_n2.y + tid)));
      if (warp_live) {
#pragma unroll
        for (int part = 0; part < H / 32; ++part) {       // 32 accumulator columns = 4 K chunks of the hidden tile at a time
          uint32_t acc[32];
          tmem_ld32(trow + part * 32, acc);
          bad |= hidden_to_smem<KEEP, BF16>(acc, s_a2 + part * 4 * kChunk, tid, relu1) && valid;
        }
      }
      tile_done(bar_r0 + 8);
      // ---- first part of the next item's encoding while layer 2 runs ----
      if (next_live)
        bad |= ladder ? encode_part1<true, BF16>(q0, mult, my_row) : encode_part1<false, BF16>(q0, mult, my_row);
      ok = __all_sync(0xffffffffu, mbar_wait(bar_b, 0u) && ok);
      tc_fence_after();
      if (!ok) break;
      if (warp_live) {                                    // layer-2 MMAs have finished reading the hidden tile
#pragma unroll
        for (int part = 0; part < H / 32; ++part) {
          uint32_t acc[32];
          tmem_ld32(trow + H + part * 32, acc);
          bad |= hidden_to_smem<KEEP, BF16>(acc, s_a2 + part * 4 * kChunk, tid, relu2) && valid;
        }
      }
      tile_done(bar_r0 + 16);
      // ---- second part of the next item's encoding while layer 3 runs ----
      if (next_live)
        bad |= ladder ? encode_part2<true, BF16>(q1, mult, my_row) : encode_part2<false, BF16>(q1, mult, my_row);
      // this item becomes the one whose output is pending; the next one becomes current
      have_prev = true;
      live_p = warp_live; valid_p = valid; decay_p = decay_c; slot_p = slot_c; relu1_p = relu1; relu2_p = relu2;
      if (!has_next) break;
      tile_done(bar_r0);
      decay_c = rec_decay(q1);
      slot_c = rec_slot(q1);
      item = next;
      wk = wk_n;
      wk_n = wk_n2;
      load_rec(wk_n, q0, q1);
      ++li;
    }
    if (ok && have_prev) {
      ok = __all_sync(0xffffffffu, mbar_wait(bar_b, 1u) && ok);
      tc_fence_after();
      if (ok) emit_output();
    }
    if (!ok && lane == 0) s_misc[1] = 1u;
    if (bad) atomicOr(status + MLPSP_ST_BITS, MLPSP_ST_NUMERIC);
  }
  tc_fence_before();
  __syncthreads();
  if (tid == 0 && s_misc[1]) atomicOr(status + MLPSP_ST_BITS, MLPSP_ST_TIMEOUT);
  if (warp == kRows / 32) tmem_free(tmem, N::kTmemCols);
}

// ------------------------------------------------------------------ small groups ----
// Work items of at most 32 records (the remainder of a primitive's records when it is small: most primitives of a
// scene with millions of primitives own a few records per wave).  A 128-row item would carry one live warp and
// three idle ones through the same chain of MMA round trips, and only five of them fit an SM.  Here one warp IS
// the CTA: the operand tiles hold 32 rows (chunk stride 512 bytes; the MMA still has M = 128 and reads, as rows
// 32..127, whatever follows -- those accumulator rows are never looked at), the accumulators of the three layers
// share 32 (H = 64: 64) columns of tensor memory, lane 0 issues the MMAs between __syncwarp()s, and 12 (6) such
// CTAs fit an SM.  Same weight pieces, same bias folding, same arithmetic as k_mlp_tc.
constexpr int kMiniRows = kRowsPerSmallItem;
constexpr int kMiniChunk = kMiniRows * 16;

template <int H>
struct MiniNet {
  using N = Net<H>;
  static constexpr int kOffConst = N::kWeightBytes;
  static constexpr int kOffA1 = kOffConst + 256;
  static constexpr int kOffA2 = kOffA1 + kA1Chunks * kMiniChunk;
  static constexpr int kOffPad = kOffA2 + (H / 8) * kMiniChunk;     // rows 32..127 of the last hidden chunk land here
  static constexpr int kOffBar = kOffPad + (kRows - kMiniRows) * 16;
  static constexpr int kSmemBytes = kOffBar + 64;                   // 17,984 (H = 32) / 33,344 (H = 64)
  static constexpr int kTmemCols = H;
  static constexpr int kCtas = H == 32 ? 12 : 6;
};

template <bool BF16, int H>
__global__ void __launch_bounds__(kMiniRows, MiniNet<H>::kCtas) k_mlp_tc_mini(
    const char* __restrict__ w16, const float* __restrict__ freq, const float* __restrict__ att,
    const float4* __restrict__ rec_in, const int4* __restrict__ work, const int32_t* __restrict__ counters,
    float4* __restrict__ rec_out, int out_mode, int32_t* __restrict__ status) {
  using N = Net<H>;
  using M = MiniNet<H>;
  chain_wait();
  chain_release();
  extern __shared__ __align__(128) char smem[];
  char* s_a1 = smem + M::kOffA1;
  char* s_a2 = smem + M::kOffA2;
  uint64_t* s_bar = reinterpret_cast<uint64_t*>(smem + M::kOffBar);   // [0..2] weight pieces, [3] MMAs of a layer done
  uint32_t* s_misc = reinterpret_cast<uint32_t*>(s_bar + 4);
  if (status[MLPSP_ST_BITS] & MLPSP_ST_FATAL) return;
  const int lane = threadIdx.x;
  const int G = counters[kCtrWorkSmall];
  int item = blockIdx.x;
  if (item >= G) return;
  const int stride = (int)gridDim.x;
  const uint32_t wb = smem_u32(smem), a1 = wb + M::kOffA1, a2 = wb + M::kOffA2;
  const uint32_t bar_w0 = smem_u32(&s_bar[0]), bar_m = smem_u32(&s_bar[3]);
  if (lane == 0) {
#pragma unroll
    for (int b = 0; b < 4; ++b) mbar_init(bar_w0 + 8 * b, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  tmem_alloc(smem_u32(&s_misc[0]), M::kTmemCols);
  if (lane < 16) {
    const uint32_t one2 = BF16 ? 0x3f803f80u : 0x3c003c00u;
    const uint32_t v = lane < 8 ? one2 : 0u;
    *reinterpret_cast<uint4*>(smem + M::kOffConst + lane * 16) = make_uint4(v, v, v, v);
  }
  // the hidden tile and the rows behind it start finite (they meet zero weights in the last layer-1 K step)
  for (int i = lane; i < (M::kOffBar - M::kOffA2) / 16; i += kMiniRows) *reinterpret_cast<uint4*>(s_a2 + i * 16) = make_uint4(0u, 0u, 0u, 0u);
  fence_async_smem();
  tc_fence_before();
  __syncwarp();
  tc_fence_after();
  const uint32_t tmem = s_misc[0];
  float mult[6];
  bool ladder = true;
#pragma unroll
  for (int f = 0; f < 6; ++f) mult[f] = __ldg(freq + f) * __ldg(att + f);
#pragma unroll
  for (int f = 1; f < 6; ++f) ladder = ladder && mult[f] == 2.0f * mult[f - 1];
  const uint64_t ones_desc = smem_desc(wb + M::kOffConst, 128, 0);
  const uint32_t idesc_h = instr_desc(kRows, H, BF16), idesc_o = instr_desc(kRows, kN3, BF16);
  const uint64_t a1_desc = smem_desc(a1, kMiniChunk, 128), a2_desc = smem_desc(a2, kMiniChunk, 128);
  const uint64_t w1_desc = smem_desc(wb + N::kOffW1, N::kWChunk, 128), w2_desc = smem_desc(wb + N::kOffW2, N::kWChunk, 128);
  const uint64_t w3_desc = smem_desc(wb + N::kOffW3, N::kW3Chunk, 128);
  auto step = [](uint64_t desc, int bytes) { return desc + (uint64_t)(bytes >> 4); };
  auto request = [&](int piece, int prim) {
    const int off = piece == 0 ? N::kOffW1 : (piece == 1 ? N::kOffW2 : N::kOffW3);
    const int bytes = piece == 0 ? N::kBytesW1 : (piece == 1 ? N::kBytesW2 : N::kBytesW3);
    mbar_expect_tx(bar_w0 + 8 * piece, bytes);
    bulk_g2s(wb + off, w16 + (size_t)prim * N::kWeightBytes + off, bytes, bar_w0 + 8 * piece);
  };
  auto load_rec = [&](const int4& w, float4& r0, float4& r1) {
    r0 = make_float4(0.f, 0.f, 0.f, 0.f);
    r1 = make_float4(0.f, 0.f, 0.f, 0.f);
    if (lane < w.z) { r0 = __ldg(rec_in + 2 * (size_t)(w.y + lane)); r1 = __ldg(rec_in + 2 * (size_t)(w.y + lane) + 1); }
  };
  // the warp's writes to an operand tile are visible to the tensor core, its reads of tensor memory have retired
  auto tile_done = [&]() {
    fence_async_smem();
    tc_fence_before();
    __syncwarp();
  };
  int4 wk = __ldg(work + item);
  int4 wk_n = (item + stride < G) ? __ldg(work + item + stride) : make_int4(0, 0, 0, 0);
  uint32_t pend = 0u;
  if (lane == 0) { request(0, wk.x); request(1, wk.x); request(2, wk.x); pend = 7u; }
  char* my_row = s_a1 + lane * 16;
  bool bad = false, ok = true;
  float4 q0, q1;
  load_rec(wk, q0, q1);
  if (ladder) { bad |= encode_part1<true, BF16, kMiniChunk>(q0, mult, my_row); bad |= encode_part2<true, BF16, kMiniChunk>(q1, mult, my_row); }
  else { bad |= encode_part1<false, BF16, kMiniChunk>(q0, mult, my_row); bad |= encode_part2<false, BF16, kMiniChunk>(q1, mult, my_row); }
  float decay_c = q1.z;
  uint32_t slot_c = __float_as_uint(q1.w);
  load_rec(wk_n, q0, q1);
  uint32_t li = 0u, ph = 0u, relu_unused = 0u;   // ph: phases of the MMA barrier completed so far
  const uint32_t trow = tmem;   // warp 0 of the CTA: lanes 0..31

  for (;;) {
    const bool valid = lane < wk.z;
    const int next = item + stride;
    const bool has_next = next < G;
    const uint32_t par = li & 1u;
    const int next2 = next + stride;
    int4 wk_n2 = make_int4(0, 0, 0, 0);
    if (next2 < G) wk_n2 = __ldg(work + next2);
    // ---- layer 1 ----
    tile_done();
    if (lane == 0) {
      bool landed = mbar_wait(bar_w0, par);
      pend &= ~1u;
      if (li == 0u) landed = landed && mbar_wait(bar_w0 + 8, 0u) && mbar_wait(bar_w0 + 16, 0u);   // see k_mlp_tc
      if (landed) {
        tc_fence_after();
#pragma unroll
        for (int ks = 0; ks < 4; ++ks)
          mma_f16(tmem, step(a1_desc, ks * 2 * kMiniChunk), step(w1_desc, ks * 2 * N::kWChunk), idesc_h, ks > 0);
        mma_f16(tmem, step(a1_desc, 8 * kMiniChunk), step(w1_desc, 8 * N::kWChunk), idesc_h, 1u);
        mma_f16(tmem, ones_desc, step(w1_desc, 10 * N::kWChunk), idesc_h, 1u);
      } else {
        ok = false;
      }
      mma_commit(bar_m);
    }
    if (next2 < G && lane < wk_n2.z) asm volatile("prefetch.global.L2 [%0];" ::"l"(rec_in + 2 * (size_t)(wk_n2.y + lane)));
    ok = __all_sync(0xffffffffu, mbar_wait(bar_m, ph++ & 1u) && ok);   // one completion per layer
    tc_fence_after();
    if (!ok) break;
    if (lane == 0 && has_next) { request(0, wk_n.x); pend |= 1u; }
#pragma unroll
    for (int part = 0; part < H / 32; ++part) {
      uint32_t acc[32];
      tmem_ld32(trow + part * 32, acc);
      bad |= hidden_to_smem<false, BF16, kMiniChunk>(acc, s_a2 + part * 4 * kMiniChunk, lane, relu_unused) && valid;
    }
    // ---- layer 2 (its accumulator takes the columns of layer 1) ----
    tile_done();
    if (lane == 0) {
      const bool landed = mbar_wait(bar_w0 + 8, par);
      pend &= ~2u;
      if (landed) {
        tc_fence_after();
#pragma unroll
        for (int ks = 0; ks < H / 16; ++ks)
          mma_f16(tmem, step(a2_desc, ks * 2 * kMiniChunk), step(w2_desc, ks * 2 * N::kWChunk), idesc_h, ks > 0);
        mma_f16(tmem, ones_desc, step(w2_desc, (H / 8) * N::kWChunk), idesc_h, 1u);
      } else {
        ok = false;
      }
      mma_commit(bar_m);
    }
    // first part of the next item's encoding while layer 2 runs (the layer-1 tile is free)
    if (has_next)
      bad |= ladder ? encode_part1<true, BF16, kMiniChunk>(q0, mult, my_row) : encode_part1<false, BF16, kMiniChunk>(q0, mult, my_row);
    ok = __all_sync(0xffffffffu, mbar_wait(bar_m, ph++ & 1u) && ok);
    tc_fence_after();
    if (!ok) break;
    if (lane == 0 && has_next) { request(1, wk_n.x); pend |= 2u; }
#pragma unroll
    for (int part = 0; part < H / 32; ++part) {
      uint32_t acc[32];
      tmem_ld32(trow + part * 32, acc);
      bad |= hidden_to_smem<false, BF16, kMiniChunk>(acc, s_a2 + part * 4 * kMiniChunk, lane, relu_unused) && valid;
    }
    // ---- layer 3 ----
    tile_done();
    if (lane == 0) {
      const bool landed = mbar_wait(bar_w0 + 16, par);
      pend &= ~4u;
      if (landed) {
        tc_fence_after();
#pragma unroll
        for (int ks = 0; ks < H / 16; ++ks)
          mma_f16(tmem, step(a2_desc, ks * 2 * kMiniChunk), step(w3_desc, ks * 2 * N::kW3Chunk), idesc_o, ks > 0);
        mma_f16(tmem, ones_desc, step(w3_desc, (H / 8) * N::kW3Chunk), idesc_o, 1u);
      } else {
        ok = false;
      }
      mma_commit(bar_m);
    }
    if (has_next)
      bad |= ladder ? encode_part2<true, BF16, kMiniChunk>(q1, mult, my_row) : encode_part2<false, BF16, kMiniChunk>(q1, mult, my_row);
    ok = __all_sync(0xffffffffu, mbar_wait(bar_m, ph++ & 1u) && ok);
    tc_fence_after();
    if (!ok) break;
    if (lane == 0 && has_next) { request(2, wk_n.x); pend |= 4u; }
    {
      uint32_t o[4];
      tmem_ld4(trow, o);
      if (valid) {
        const float o0 = __uint_as_float(o[0]), o1 = __uint_as_float(o[1]), o2 = __uint_as_float(o[2]), o3 = __uint_as_float(o[3]);
        const float sigma_raw = softplus_fast(o3);
        float4 out;
        out.x = sigmoid_fast(o0); out.y = sigmoid_fast(o1); out.z = sigmoid_fast(o2);
        out.w = (out_mode == kOutAlpha) ? (1.f - __expf(-(sigma_raw * decay_c))) : sigma_raw;
        rec_out[slot_c] = out;
      }
    }
    if (!has_next) break;
    decay_c = q1.z;
    slot_c = __float_as_uint(q1.w);
    item = next;
    wk = wk_n;
    wk_n = wk_n2;
    load_rec(wk_n, q0, q1);
    ++li;
  }
  if (!ok && lane == 0) {
    atomicOr(status + MLPSP_ST_BITS, MLPSP_ST_TIMEOUT);
    for (int b = 0; b < 3; ++b)
      if (pend & (1u << b)) mbar_wait(bar_w0 + 8 * b, li & 1u);
  }
  if (bad) atomicOr(status + MLPSP_ST_BITS, MLPSP_ST_NUMERIC);
  tc_fence_before();
  __syncwarp();
  tmem_free(tmem, M::kTmemCols);
}

// ------------------------------------------------------------------------------ packing ----
template <bool BF16>
__device__ __forceinline__ uint16_t to_lp(float x, bool& bad) {
  if (BF16) {
    const __nv_bfloat16 v = __float2bfloat16_rn(x);
    bad |= __hisinf(v) || __hisnan(v);
    return *reinterpret_cast<const uint16_t*>(&v);
  }
  const __half v = __float2half_rn(x);
  bad |= __hisinf(v) || __hisnan(v);
  return *reinterpret_cast<const uint16_t*>(&v);
}
template <bool BF16>
__device__ __forceinline__ float from_lp(uint16_t u) {
  if (BF16) return __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(&u));
  return __half2float(*reinterpret_cast<const __half*>(&u));
}

// A bias as a sum of up to eight operand-format terms (greedy: each term is the remainder clamped to the
// format's range and rounded): three terms carry every FP32 mantissa bit, the others serve biases beyond the
// format's range (8 x 65504 for binary16).  A bias that does not fit is reported.
template <bool BF16>
__device__ __forceinline__ void bias_terms(float b, uint16_t* dst /* [8] */, bool& bad) {
  const float lim = BF16 ? 3.3e38f : 65504.f;
  float rem = b;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    bool ignore = false;
    const uint16_t t = to_lp<BF16>(fminf(fmaxf(rem, -lim), lim), ignore);
    dst[j] = (rem == rem) ? t : (uint16_t)0;
    if (rem == rem) rem -= from_lp<BF16>(t);
  }
  bad |= !(fabsf(rem) <= 1e-6f * fabsf(b) + 1e-7f);
}

template <bool BF16, int H>
__global__ void k_pack_weights(const float* __restrict__ W1, const float* __restrict__ b1, const float* __restrict__ W2,
                               const float* __restrict__ b2, const float* __restrict__ W3, const float* __restrict__ b3,
                               int n, char* __restrict__ out, int32_t* __restrict__ status) {
  const int p = blockIdx.x;
  if (p >= n) return;
  using N = Net<H>;
  char* dst = out + (size_t)p * N::kWeightBytes;
  uint16_t* w1 = reinterpret_cast<uint16_t*>(dst + N::kOffW1);
  uint16_t* w2 = reinterpret_cast<uint16_t*>(dst + N::kOffW2);
  uint16_t* w3 = reinterpret_cast<uint16_t*>(dst + N::kOffW3);
  bool bad = false;
  for (int i = threadIdx.x; i < H * 80; i += blockDim.x) {
    const int h = i / 80, k = i % 80;                   // k >= 72: the zero chunk
    const uint16_t v = to_lp<BF16>(k < 72 ? W1[(size_t)p * H * 72 + h * 72 + k] : 0.f, bad);
    const int kk = enc_k_of_reference(k);
    w1[(kk >> 3) * (H * 8) + h * 8 + (kk & 7)] = v;
  }
  for (int i = threadIdx.x; i < H * H; i += blockDim.x) {
    const int h = i / H, k = i % H;
    const uint16_t v = to_lp<BF16>(W2[(size_t)p * H * H + i], bad);
    w2[(k >> 3) * (H * 8) + h * 8 + (k & 7)] = v;
  }
  for (int i = threadIdx.x; i < kN3 * H; i += blockDim.x) {
    const int h = i / H, k = i % H;
    const uint16_t v = to_lp<BF16>(h < 4 ? W3[(size_t)p * 4 * H + h * H + k] : 0.f, bad);
    w3[(k >> 3) * (kN3 * 8) + h * 8 + (k & 7)] = v;
  }
  for (int h = threadIdx.x; h < H; h += blockDim.x) {
    bias_terms<BF16>(b1[(size_t)p * H + h], w1 + 10 * (H * 8) + h * 8, bad);
    bias_terms<BF16>(b2[(size_t)p * H + h], w2 + (H / 8) * (H * 8) + h * 8, bad);
  }
  for (int h = threadIdx.x; h < kN3; h += blockDim.x) {
    uint16_t* row = w3 + (H / 8) * (kN3 * 8) + h * 8;
    if (h < 4) bias_terms<BF16>(b3[(size_t)p * 4 + h], row, bad);
    else for (int j = 0; j < 8; ++j) row[j] = 0;
  }
  if (bad && status) atomicOr(status + MLPSP_ST_BITS, MLPSP_ST_NUMERIC);
}

template <bool KEEP, bool BF16, int H>
static int launch_one(const char* image, const mlpsp_scene* sc, const RecIn* rec_in, const int4* work, const int32_t* counters,
                      float4* rec_out, float4* rec_ext, int out_mode, int32_t* status, cudaStream_t st, int grid) {
  using N = Net<H>;
  static DeviceOnce attr_once;
  if (attr_once.first())
    MLPSP_CUDA_OK(cudaFuncSetAttribute(k_mlp_tc<KEEP, BF16, H>, cudaFuncAttributeMaxDynamicSharedMemorySize, N::kSmemBytes));
  launch_chained(k_mlp_tc<KEEP, BF16, H>, dim3(grid), dim3(kMlpThreads), N::kSmemBytes, st, image, sc->freq, sc->att, reinterpret_cast<const float4*>(rec_in),
                                                                   work, counters, rec_out, rec_ext, out_mode, status);
  return MLPSP_OK;
}

template <bool BF16, int H>
static int launch_mini(const char* image, const mlpsp_scene* sc, const RecIn* rec_in, const int4* work_small,
                       const int32_t* counters, float4* rec_out, int out_mode, int32_t* status, cudaStream_t st, int grid) {
  using M = MiniNet<H>;
  static DeviceOnce attr_once;
  if (attr_once.first())
    MLPSP_CUDA_OK(cudaFuncSetAttribute(k_mlp_tc_mini<BF16, H>, cudaFuncAttributeMaxDynamicSharedMemorySize, M::kSmemBytes));
  launch_chained(k_mlp_tc_mini<BF16, H>, dim3(grid), dim3(kMiniRows), M::kSmemBytes, st, image, sc->freq, sc->att, reinterpret_cast<const float4*>(rec_in),
                                                                work_small, counters, rec_out, out_mode, status);
  return MLPSP_OK;
}

template <int H>
static int launch_tc(const mlpsp_scene* sc, const char* image, const RecIn* rec_in, const int4* work, const int4* work_small,
                     const int32_t* counters, float4* rec_out, float4* rec_ext, int out_mode, int32_t* status, cudaStream_t st,
                     bool bf16, int grid_cap) {
  using N = Net<H>;
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  int grid = sms * N::kCtas;
  if (grid_cap > 0) grid = std::min(grid, grid_cap);
  LaunchScope scope(kKMlp, (work_small && !rec_ext) ? 2 : 1, st);
  int rc;
  if (rec_ext) {
    if (H != 32) {
      set_error("record export needs hidden width 32 (32-bit ReLU masks)");
      return MLPSP_E_LIMIT;
    }
    rc = bf16 ? launch_one<true, true, 32>(image, sc, rec_in, work, counters, rec_out, rec_ext, out_mode, status, st, grid)
              : launch_one<true, false, 32>(image, sc, rec_in, work, counters, rec_out, rec_ext, out_mode, status, st, grid);
  } else {
    rc = bf16 ? launch_one<false, true, H>(image, sc, rec_in, work, counters, rec_out, rec_ext, out_mode, status, st, grid)
              : launch_one<false, false, H>(image, sc, rec_in, work, counters, rec_out, rec_ext, out_mode, status, st, grid);
  }
  if (rc) return rc;
  if (work_small && !rec_ext) {
    // the wave's small groups (at most 32 records) on their own kernel: one warp per item, twelve (six) items per SM
    int grid_s = sms * MiniNet<H>::kCtas;
    if (grid_cap > 0) grid_s = std::min(grid_s, grid_cap);
    rc = bf16 ? launch_mini<true, H>(image, sc, rec_in, work_small, counters, rec_out, out_mode, status, st, grid_s)
              : launch_mini<false, H>(image, sc, rec_in, work_small, counters, rec_out, out_mode, status, st, grid_s);
    if (rc) return rc;
  }
  return cuda_check(cudaGetLastError(), "mlp_f16");
}

int launch_mlp_f16(const mlpsp_scene* sc, const RecIn* rec_in, const int32_t* prim_off, const int4* work,
                   const int32_t* counters, float4* rec_out, float4* rec_ext, int out_mode, int32_t* status,
                   cudaStream_t st, bool bf16, int grid_cap, const int4* work_small) {
  MLPSP_REQUIRE((sc->hidden == 32 || sc->hidden == 64) && sc->num_freq == 6, MLPSP_E_LIMIT,
                "the tensor-core evaluator is built for 72->H->H->4 networks with H = 32 or 64 (6 frequencies)");
  const char* image = (const char*)(bf16 ? sc->wbf16 : sc->w16);
  MLPSP_REQUIRE(image && sc->freq && sc->att, MLPSP_E_ARG, "%s evaluator needs the packed weight image",
                bf16 ? "bf16" : "fp16");
  MLPSP_REQUIRE((reinterpret_cast<uintptr_t>(image) & 15) == 0, MLPSP_E_ARG, "the packed weight image must be 16-byte aligned");
  (void)prim_off;
  if (sc->hidden == 64)
    return launch_tc<64>(sc, image, rec_in, work, work_small, counters, rec_out, rec_ext, out_mode, status, st, bf16, grid_cap);
  return launch_tc<32>(sc, image, rec_in, work, work_small, counters, rec_out, rec_ext, out_mode, status, st, bf16, grid_cap);
}

}  // namespace mlpsp

using namespace mlpsp;

extern "C" int64_t mlpsp_packed_weight_bytes(int32_t hidden, int32_t num_freq) {
  if (num_freq != 6) return 0;
  return hidden == 32 ? Net<32>::kWeightBytes : (hidden == 64 ? Net<64>::kWeightBytes : 0);
}

static int pack_weights(const mlpsp_scene* sc, void* out, int32_t* status, void* stream, bool bf16, const char* who) {
  MLPSP_REQUIRE(sc && out, MLPSP_E_ARG, "%s: null pointer", who);
  MLPSP_REQUIRE((sc->hidden == 32 || sc->hidden == 64) && sc->num_freq == 6, MLPSP_E_LIMIT,
                "%s: only 72->H->H->4 networks with H = 32 or 64 have a packed image", who);
  MLPSP_REQUIRE(sc->W1 && sc->b1 && sc->W2 && sc->b2 && sc->W3 && sc->b3, MLPSP_E_ARG, "%s: FP32 weights missing", who);
  if (sc->n == 0) return MLPSP_OK;
  cudaStream_t st = (cudaStream_t)stream;
  LaunchScope scope(kKMisc, 1, st);
#define MLPSP_PACK(BF, HH)                                                                                         \
  k_pack_weights<BF, HH><<<sc->n, 128, 0, st>>>(sc->W1, sc->b1, sc->W2, sc->b2, sc->W3, sc->b3, sc->n, (char*)out, status)
  if (sc->hidden == 64) { if (bf16) MLPSP_PACK(true, 64); else MLPSP_PACK(false, 64); }
  else { if (bf16) MLPSP_PACK(true, 32); else MLPSP_PACK(false, 32); }
#undef MLPSP_PACK
  return cuda_check(cudaGetLastError(), who);
}

extern "C" int mlpsp_pack_weights_f16(const mlpsp_scene* sc, void* w16_out, int32_t* status, void* stream) {
  return pack_weights(sc, w16_out, status, stream, false, "mlpsp_pack_weights_f16");
}

extern "C" int mlpsp_pack_weights_bf16(const mlpsp_scene* sc, void* wbf16_out, int32_t* status, void* stream) {
  return pack_weights(sc, wbf16_out, status, stream, true, "mlpsp_pack_weights_bf16");
}
