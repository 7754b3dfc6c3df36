// Persistent bidirectional GRU layer for sm_100a (see gru_persistent.h for the interface).
//
// Work split. Direction d of a layer is run by H/16 blocks (grid.y = direction); block c owns
// the hidden units [16c, 16c+16). Forward, it keeps the 48 rows of W_hh that produce the r, z and
// n pre-activations of its units (48 x H fp32 = 192 KiB at H = 1024) in shared memory for the
// whole sequence. Each time step it
//   1. waits until every block of its direction has published h_{t-1} (a counter in global
//      memory, release/acquire at gpu scope, bounded wait),
//   2. streams h_{t-1} (B x H) through two 16 KiB shared-memory stages with TMA
//      (cp.async.bulk.tensor, 128-byte swizzle) while one thread issues tcgen05.mma (TF32
//      operands, M = 128 rows of which 48 are weights, N = 32 batch columns, K = 8 per
//      instruction) into a 32-column accumulator in tensor memory,
//   3. reads the accumulator back (tcgen05.ld), applies the gate non-linearities for its 16 units,
//      writes h_t into the layer output and the saved activations, and signals the counter.
// Backward, the block holds the 16 rows of W_hh^T that belong to its units (16 x 3H) and each
// step first turns dh_t into the pre-activation gradients of its units, publishes them, and then
// multiplies the full (B x 3H) pre-activation gradient by its weight rows to obtain the recurrent
// part of dh_{t-1} for its units.
//
// The MMA always reads 128 operand rows starting at a tile's base; rows past the block's own
// weight rows alias whatever follows in shared memory and only produce accumulator rows that
// are never read. All shared-memory offsets keep those reads inside the allocation.
//
// Every wait (mbarrier, step counter) is bounded by %globaltimer. When a wait runs out the block
// records a status bit, waits (bounded) for its own copies and MMAs in flight, frees its tensor
// memory and returns.
#include "gru_persistent.h"

#include <cuda.h>

#include <algorithm>
#include <mutex>

namespace bc {
namespace gpu {

namespace {

constexpr int kUnits = 16;            // hidden units per block
constexpr int kBatchTile = 32;        // MMA N and rows of one TMA box of the streamed operand
constexpr int kKTile = 32;            // fp32 elements in one 128-byte swizzle row
constexpr int kTilesPerStage = 4;     // K tiles per pipeline stage (K = 128)
constexpr int kStageBytes = kTilesPerStage * kBatchTile * 128;   // 16 KiB
constexpr int kXTileBytes = kBatchTile * 128;                    // 4 KiB
constexpr int kThreads = 128;
constexpr int kAccumulators = 4;     // independent accumulators, summed in the epilogue (see drive_product)
constexpr int kTmemCols = kAccumulators * kBatchTile;
constexpr int kGStride = 33;          // padded row of the accumulator copy in shared memory
constexpr int kMmaM = 128;

struct Params {
  GruDims d;
  const float* b_hh;    // forward
  const float* gx;      // forward
  float* y;             // forward: out; backward: in (const)
  float* rsv;           // forward: out; backward: in
  const float* dy;      // backward
  float* dgx;           // backward
  float* dgh;           // backward
  uint32_t* sync;
  uint32_t* status;
  unsigned long long timeout_ns;
  unsigned long long* prof;   // optional: 8 time stamps per step of block (0, 0), for tuning
  int debug;                  // tuning only: 1 = issue no MMA, 2 = issue no operand copies (results are then wrong)
};

// ---- PTX wrappers ---------------------------------------------------------------------------

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ unsigned long long gtimer() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}
// Bounded wait for the phase with the given parity; also gives up when `abort_flag` is raised.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, unsigned long long timeout_ns, const volatile int* abort_flag) {
  if (mbar_try_wait(bar, parity)) return true;
  const unsigned long long t0 = gtimer();
  uint32_t spins = 0;
  while (!mbar_try_wait(bar, parity)) {
    if (abort_flag) __nanosleep(64);   // the many waiting threads leave the issue slots to the driver
    if (((++spins) & 63) == 0) {
      if (abort_flag && *abort_flag) return false;
      if (gtimer() - t0 > timeout_ns) return false;
    }
  }
  return true;
}
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async;" ::: "memory"); }
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_mma_tf32(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
// Same with the accumulate input always enabled (no predicate set-up).
__device__ __forceinline__ void tc_mma_tf32_acc(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.eq.u32 p, 1, 1;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc) : "memory");
}
__device__ __forceinline__ void tc_ld32(uint32_t taddr, float* v) {
  uint32_t r[32];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
        "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
        "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr) : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 32; i++) v[i] = __uint_as_float(r[i]);
}

// Sum of the kAccumulators accumulators (32 columns each) for this thread's lane.
__device__ __forceinline__ void tc_ld32_sum(uint32_t taddr, float* v);

// Shared-memory matrix descriptor of a K-major operand tile stored as rows of 128 bytes with the
// 128-byte swizzle (what TMA writes for a box that is 32 fp32 wide): groups of 8 rows are 1024
// bytes apart; the leading-dimension offset is unused because a tile is one swizzle atom wide.
__device__ __forceinline__ uint64_t operand_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);   // start address
  d |= (uint64_t)(1024u >> 4) << 32;              // stride between 8-row groups
  d |= (uint64_t)1 << 46;                         // descriptor version of sm_100
  d |= (uint64_t)2 << 61;                         // 128-byte swizzle
  return d;
}

// kind::tf32, fp32 accumulator, both operands K-major, M x N = 128 x 32.
constexpr uint32_t kInstrDesc = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(kBatchTile >> 3) << 17) | ((uint32_t)(kMmaM >> 4) << 24);

__device__ __forceinline__ void tc_ld32_sum(uint32_t taddr, float* v) {
  tc_ld32(taddr, v);
#pragma unroll
  for (int a = 1; a < kAccumulators; a++) {
    float w[32];
    tc_ld32(taddr + a * kBatchTile, w);
#pragma unroll
    for (int i = 0; i < 32; i++) v[i] += w[i];
  }
}

__device__ __forceinline__ float sigmoidf_(float x) { return 1.f / (1.f + __expf(-x)); }

__device__ __forceinline__ bool wait_counter(const uint32_t* ctr, uint32_t target, unsigned long long timeout_ns) {
  const unsigned long long t0 = gtimer();
  uint32_t spins = 0;
  for (;;) {
    uint32_t v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(ctr) : "memory");
    if ((int32_t)(v - target) >= 0) return true;
    if (((++spins) & 31) == 0 && gtimer() - t0 > timeout_ns) return false;
  }
}
__device__ __forceinline__ void signal_counter(uint32_t* ctr) {
  asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(ctr) : "memory");
}

// State of the one thread per block that issues copies and MMAs.
struct Driver {
  uint32_t full_phase[2];
  uint32_t empty_phase[2];
  bool pending[2];
};

// One recurrent product: wait for the peers' data of this step, stream the (32 x K) operand
// through the two stages and accumulate D = W_rows x X^T in tensor memory. Thread 0 only.
// `row0` is the first row of the streamed operand in its tensor map, `col0` its first column.
__device__ __forceinline__ uint32_t drive_product(Driver& dr, const CUtensorMap* tm_x, int row0, int col0, int nchunks, uint32_t w_addr,
                                                  int w_tile_bytes, uint32_t x_addr, uint32_t bars, uint32_t tmem, const uint32_t* ctr,
                                                  uint32_t target, unsigned long long timeout_ns, unsigned long long* stamp, int debug) {
  const uint32_t full0 = bars, empty0 = bars + 16, done = bars + 32;
  const int rot = (int)(blockIdx.x % (unsigned)nchunks);
  const uint64_t a_desc0 = operand_desc(w_addr), b_desc0 = operand_desc(x_addr);
  if (!wait_counter(ctr, target, timeout_ns)) return kGruTimeoutGrid;
  if (stamp) stamp[1] = gtimer();
  fence_proxy_async();   // peers wrote the operand with ordinary stores; TMA reads it through the async proxy
  // Every block of a direction streams the same operand. Each starts at a different K chunk
  // (`rot`) and wraps around, so that at any moment the blocks read different lines of L2
  // instead of all asking the same few slices for the same lines.
  auto load_chunk = [&](int c) {
    if (debug & 2) return;
    const int st = c & 1;
    int kc = c + rot;
    if (kc >= nchunks) kc -= nchunks;
    mbar_expect_tx(full0 + 8 * st, kStageBytes);
    dr.pending[st] = true;
#pragma unroll
    for (int i = 0; i < kTilesPerStage; i++)
      tma_load_2d(x_addr + st * kStageBytes + i * kXTileBytes, tm_x, col0 + (kc * kTilesPerStage + i) * kKTile, row0, full0 + 8 * st);
  };
  load_chunk(0);
  if (nchunks > 1) load_chunk(1);
  for (int c = 0; c < nchunks; c++) {
    const int st = c & 1;
    int kc = c + rot;
    if (kc >= nchunks) kc -= nchunks;
    if (!(debug & 2)) {
      if (!mbar_wait(full0 + 8 * st, dr.full_phase[st], timeout_ns, nullptr)) return kGruTimeoutCopy;
      dr.full_phase[st] ^= 1;
      dr.pending[st] = false;
    }
    if (stamp && c == 0) stamp[2] = gtimer();
    tc_fence_after();
    // One thread issues every MMA of the step and each MMA is small (N = 32), so the issue path is
    // kept to a few instructions: descriptors differ from a per-chunk base only in their address
    // field (bits 0-13, in units of 16 bytes), which cannot carry into the next field because all
    // addresses lie below 256 KiB.
    // Consecutive MMAs into one accumulator form a dependent chain whose per-link latency (about
    // 120 clocks, measured) is far above the work of one N = 32 MMA, so the four K steps of a tile
    // go to four different accumulators; the epilogue adds them up.
    if (!(debug & 1)) {
    const uint64_t a_base = a_desc0 + (uint64_t)(((uint32_t)kc * kTilesPerStage * (uint32_t)w_tile_bytes) >> 4);
    const uint64_t b_base = b_desc0 + (uint64_t)((st * kStageBytes) >> 4);
    if (c == 0) {
#pragma unroll
      for (int ks = 0; ks < 4; ks++) tc_mma_tf32(tmem + ks * kBatchTile, a_base + 2 * ks, b_base + 2 * ks, kInstrDesc, 0u);
    } else {
#pragma unroll
      for (int ks = 0; ks < 4; ks++) tc_mma_tf32_acc(tmem + ks * kBatchTile, a_base + 2 * ks, b_base + 2 * ks, kInstrDesc);
    }
#pragma unroll
    for (int i = 1; i < kTilesPerStage; i++) {
      const uint64_t a_i = a_base + (uint64_t)((i * w_tile_bytes) >> 4);
      const uint64_t b_i = b_base + (uint64_t)((i * kXTileBytes) >> 4);
#pragma unroll
      for (int ks = 0; ks < 4; ks++) tc_mma_tf32_acc(tmem + ks * kBatchTile, a_i + 2 * ks, b_i + 2 * ks, kInstrDesc);
    }
    }
    if (c + 2 < nchunks) {
      // Refill this stage as soon as its MMAs have read it, so that two copies are always in
      // flight: the stream is bound by copy latency, not by the tensor core.
      tc_commit(empty0 + 8 * st);
      if (!mbar_wait(empty0 + 8 * st, dr.empty_phase[st], timeout_ns, nullptr)) return kGruTimeoutMma;
      dr.empty_phase[st] ^= 1;
      load_chunk(c + 2);
    }
  }
  tc_commit(done);
  if (stamp) stamp[3] = gtimer();
  return 0;
}

// Inputs of one backward step for the (unit, batch) pairs of a thread.
struct BwdInputs {
  float r[4], z[4], n[4], hn[4], hp[4], dy[4];
};

__device__ __forceinline__ void load_bwd_inputs(const Params& p, BwdInputs& in, int t, int dir, int unit, int bq) {
  const int T = p.d.T, B = p.d.B, H = p.d.H, ND = p.d.ndir;
  const int tprev = dir ? t + 1 : t - 1;
  const bool has_prev = tprev >= 0 && tprev < T;
#pragma unroll
  for (int j = 0; j < 4; j++) {
    const int b = bq + 8 * j;
    if (b < B) {
      const float* rs = p.rsv + (((size_t)(dir * T + t) * B + b) * 4) * H + unit;
      in.r[j] = rs[0]; in.z[j] = rs[H]; in.n[j] = rs[2 * H]; in.hn[j] = rs[3 * H];
      in.hp[j] = has_prev ? p.y[((size_t)tprev * B + b) * (ND * H) + dir * H + unit] : 0.f;
      in.dy[j] = p.dy[((size_t)t * B + b) * (ND * H) + dir * H + unit];
    }
  }
}

template <bool BWD>
__global__ void __launch_bounds__(kThreads, 1) gru_persistent_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_x,
                                                                      const __grid_constant__ Params p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  uint8_t* smem = smem_raw + ((1024u - (raw_addr & 1023u)) & 1023u);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int dir = blockIdx.y, u0 = blockIdx.x * kUnits;
  const int T = p.d.T, B = p.d.B, H = p.d.H, ND = p.d.ndir;
  const int nblocks = gridDim.x;
  const int kdim = BWD ? 3 * H : H;
  constexpr int kRows = BWD ? kUnits : 3 * kUnits;
  constexpr int kWTile = kRows * 128;
  const int nkt = kdim / kKTile;
  const int nchunks = kdim / (kKTile * kTilesPerStage);

  uint8_t* w_s = smem;
  uint8_t* x_s = smem + (size_t)nkt * kWTile;
  float* g_s = reinterpret_cast<float*>(x_s);   // accumulator copy; aliases stage 0 between products
  uint64_t* bar_s = reinterpret_cast<uint64_t*>(x_s + 2 * kStageBytes);   // full[2], empty[2], done, weights
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_s + 6);
  volatile int* abort_s = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const uint32_t bars = smem_u32(bar_s);
  const uint32_t done_bar = bars + 32, w_bar = bars + 40;

  if (tid == 0) {
    for (int i = 0; i < 6; i++) mbar_init(bars + 8 * i, 1);
    *abort_s = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  // The block's weight rows: loaded once, resident for the whole sequence.
  if (tid == 0) {
    mbar_expect_tx(w_bar, (uint32_t)(nkt * kWTile));
    for (int kt = 0; kt < nkt; kt++) {
      if (BWD) {
        tma_load_2d(smem_u32(w_s) + kt * kWTile, &tm_w, kt * kKTile, dir * H + u0, w_bar);
      } else {
        for (int g = 0; g < 3; g++)
          tma_load_2d(smem_u32(w_s) + kt * kWTile + g * (kUnits * 128), &tm_w, kt * kKTile, dir * 3 * H + g * H + u0, w_bar);
      }
    }
  }
  bool ok = mbar_wait(w_bar, 0, p.timeout_ns, nullptr);
  if (!ok && tid == 0) atomicOr(p.status, kGruTimeoutCopy);
  ok = __syncthreads_and(ok) != 0;

  Driver dr;
  dr.full_phase[0] = dr.full_phase[1] = dr.empty_phase[0] = dr.empty_phase[1] = 0;
  dr.pending[0] = dr.pending[1] = false;
  uint32_t done_phase = 0;
  bool mma_in_flight = false;

  // Thread (u, bq) handles unit u0 + u for the batch entries bq, bq + 8, bq + 16, bq + 24.
  const int u = tid & 15, bq = tid >> 4;
  float carry[4] = {0.f, 0.f, 0.f, 0.f};   // forward: h_{t-1}; backward: recurrent part of dh_t
  float bias_r = 0.f, bias_z = 0.f, bias_n = 0.f;
  if (!BWD) {
    bias_r = p.b_hh[dir * 3 * H + u0 + u];
    bias_z = p.b_hh[dir * 3 * H + H + u0 + u];
    bias_n = p.b_hh[dir * 3 * H + 2 * H + u0 + u];
  }
  uint32_t* ctr = p.sync + dir;
  BwdInputs pre;

  for (int s = 0; ok && s < T; s++) {
    uint32_t fail = 0;
    unsigned long long* stamp = (p.prof && tid == 0 && blockIdx.x == 0 && blockIdx.y == 0) ? p.prof + (size_t)s * 8 : nullptr;
    if (stamp) stamp[0] = gtimer();
    if (!BWD) {
      // ---------------- forward step ----------------
      const int t = dir ? T - 1 - s : s;
      const int tprev = dir ? t + 1 : t - 1;
      float gxr[4], gxz[4], gxn[4];
#pragma unroll
      for (int j = 0; j < 4; j++) {
        const int b = bq + 8 * j;
        if (b < B) {
          const float* g = p.gx + (((size_t)t * B + b) * ND + dir) * 3 * H + u0 + u;
          gxr[j] = g[0]; gxz[j] = g[H]; gxn[j] = g[2 * H];
        }
      }
      if (s > 0) {
        if (tid == 0) {
          fail = drive_product(dr, &tm_x, tprev * B, dir * H, nchunks, smem_u32(w_s), kWTile, smem_u32(x_s), bars, tmem, ctr,
                               (uint32_t)nblocks * (uint32_t)s, p.timeout_ns, stamp, p.debug);
          if (fail) { atomicOr(p.status, fail); *abort_s = 1; }
        }
        __syncwarp();
        bool got = mbar_wait(done_bar, done_phase, 4 * p.timeout_ns, abort_s);
        got = __all_sync(0xffffffffu, got) != 0;
        if (got) done_phase ^= 1;
        if (stamp) stamp[4] = gtimer();
        tc_fence_after();
        if (got && warp < 2) {
          float v[32];
          tc_ld32_sum(tmem + ((uint32_t)(warp * 32) << 16), v);
          const int row = warp * 32 + lane;
          if (row < kRows) {
#pragma unroll
            for (int c = 0; c < 32; c++) g_s[row * kGStride + c] = v[c];
          }
        }
        tc_fence_before();
        ok = __syncthreads_and(got && !fail) != 0;
        if (!ok) { mma_in_flight = true; break; }
      }
#pragma unroll
      for (int j = 0; j < 4; j++) {
        const int b = bq + 8 * j;
        if (b < B) {
          float hr = bias_r, hz = bias_z, hn = bias_n;
          if (s > 0) {
            hr += g_s[u * kGStride + b];
            hz += g_s[(kUnits + u) * kGStride + b];
            hn += g_s[(2 * kUnits + u) * kGStride + b];
          }
          const float r = sigmoidf_(gxr[j] + hr);
          const float z = sigmoidf_(gxz[j] + hz);
          const float n = tanhf(gxn[j] + r * hn);
          const float h = n + z * (carry[j] - n);
          carry[j] = h;
          p.y[((size_t)t * B + b) * (ND * H) + dir * H + u0 + u] = h;
          float* rs = p.rsv + (((size_t)(dir * T + t) * B + b) * 4) * H + u0 + u;
          rs[0] = r; rs[H] = z; rs[2 * H] = n; rs[3 * H] = hn;
        }
      }
      if (stamp) stamp[5] = gtimer();
      if (s + 1 < T) {
        __threadfence();
        fence_proxy_async();
        __syncthreads();
        if (tid == 0) signal_counter(ctr);
      }
      if (stamp) stamp[6] = gtimer();
    } else {
      // ---------------- backward step ----------------
      const int t = dir ? s : T - 1 - s;
      if (s == 0) load_bwd_inputs(p, pre, t, dir, u0 + u, bq);
      float keep[4];
#pragma unroll
      for (int j = 0; j < 4; j++) {
        const int b = bq + 8 * j;
        keep[j] = 0.f;
        if (b < B) {
          const float r = pre.r[j], z = pre.z[j], n = pre.n[j], hn = pre.hn[j], hp = pre.hp[j];
          const float dh = pre.dy[j] + carry[j];
          const float dn = dh * (1.f - z) * (1.f - n * n);
          const float dz = dh * (hp - n) * z * (1.f - z);
          const float drr = dn * hn * r * (1.f - r);
          const size_t o = (((size_t)t * B + b) * ND + dir) * 3 * H + u0 + u;
          p.dgx[o] = drr; p.dgx[o + H] = dz; p.dgx[o + 2 * H] = dn;
          p.dgh[o] = drr; p.dgh[o + H] = dz; p.dgh[o + 2 * H] = dn * r;
          keep[j] = dh * z;
        }
      }
      if (stamp) stamp[5] = gtimer();
      if (s + 1 < T) {
        __threadfence();
        fence_proxy_async();
        __syncthreads();
        // Next step's saved activations and output gradient: in flight while the product runs.
        load_bwd_inputs(p, pre, dir ? s + 1 : T - 2 - s, dir, u0 + u, bq);
        if (tid == 0) {
          signal_counter(ctr);
          if (stamp) stamp[6] = gtimer();
          fail = drive_product(dr, &tm_x, t * B, dir * 3 * H, nchunks, smem_u32(w_s), kWTile, smem_u32(x_s), bars, tmem, ctr,
                               (uint32_t)nblocks * (uint32_t)(s + 1), p.timeout_ns, stamp, p.debug);
          if (fail) { atomicOr(p.status, fail); *abort_s = 1; }
        }
        __syncwarp();
        bool got = mbar_wait(done_bar, done_phase, 4 * p.timeout_ns, abort_s);
        got = __all_sync(0xffffffffu, got) != 0;
        if (got) done_phase ^= 1;
        if (stamp) stamp[4] = gtimer();
        tc_fence_after();
        if (got && warp == 0) {
          float v[32];
          tc_ld32_sum(tmem, v);
          if (lane < kRows) {
#pragma unroll
            for (int c = 0; c < 32; c++) g_s[lane * kGStride + c] = v[c];
          }
        }
        tc_fence_before();
        ok = __syncthreads_and(got && !fail) != 0;
        if (!ok) { mma_in_flight = true; break; }
#pragma unroll
        for (int j = 0; j < 4; j++) {
          const int b = bq + 8 * j;
          carry[j] = b < B ? keep[j] + g_s[u * kGStride + b] : 0.f;
        }
        tc_fence_before();
        __syncthreads();   // g_s (stage 0) is overwritten by the next product's first copy
      }
    }
  }

  // Leave cleanly: nothing of this block may still be in flight when tensor memory is freed.
  if (tid == 0 && (mma_in_flight || !ok)) {
    for (int st = 0; st < 2; st++)
      if (dr.pending[st]) mbar_wait(bars + 8 * st, dr.full_phase[st], p.timeout_ns, nullptr);
    tc_commit(done_bar);
    mbar_wait(done_bar, done_phase, p.timeout_ns, nullptr);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    __syncwarp();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
  }
}

// ---- host side ------------------------------------------------------------------------------

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
    else
      (void)cudaGetLastError();
  });
  return fn;
}

// Row-major fp32 matrix [rows, cols] viewed in boxes of `box_rows` x 32 columns, 128-byte swizzle.
bool make_map(CUtensorMap* m, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t gdim[2] = {cols, rows};
  cuuint64_t gstride[1] = {cols * sizeof(float)};
  cuuint32_t box[2] = {(cuuint32_t)kKTile, box_rows};
  cuuint32_t estr[2] = {1, 1};
  return fn(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void*>(base), gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

unsigned long long* g_prof = nullptr;   // set by gru_persistent_set_profile()
int g_debug = 0;

size_t smem_bytes(const GruDims& d, bool bwd) {
  const size_t kdim = bwd ? 3 * (size_t)d.H : (size_t)d.H;
  const size_t rows = bwd ? kUnits : 3 * kUnits;
  return (kdim / kKTile) * rows * 128 + 2 * kStageBytes + 128 + 1024;
}

bool dims_ok(const GruDims& d) {
  return d.T >= 1 && d.B >= 1 && d.B <= kBatchTile && d.H >= 128 && d.H <= 1024 && d.H % 128 == 0 && (d.ndir == 1 || d.ndir == 2);
}

bool aligned16(const void* p) { return ((uintptr_t)p & 15) == 0; }

template <bool BWD>
cudaError_t launch(const GruDims& d, const CUtensorMap& tm_w, const CUtensorMap& tm_x, const Params& p, cudaStream_t stream) {
  const size_t smem = smem_bytes(d, BWD);
  auto kernel = gru_persistent_kernel<BWD>;
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  int dev = 0, sms = 0, per_sm = 0;
  if ((e = cudaGetDevice(&dev)) != cudaSuccess) return e;
  if ((e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev)) != cudaSuccess) return e;
  if ((e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, kThreads, smem)) != cudaSuccess) return e;
  dim3 grid(d.H / kUnits, d.ndir), block(kThreads);
  if ((int)(grid.x * grid.y) > per_sm * sms) return cudaErrorCooperativeLaunchTooLarge;
  void* args[] = {(void*)&tm_w, (void*)&tm_x, (void*)&p};
  return cudaLaunchCooperativeKernel((const void*)kernel, grid, block, args, smem, stream);
}

}  // namespace

void gru_persistent_set_profile(unsigned long long* stamps) { g_prof = stamps; }
void gru_persistent_set_debug(int flags) { g_debug = flags; }

bool gru_persistent_supported(const GruDims& d, int device) {
  if (!dims_ok(d) || !encode_fn()) return false;
  int major = 0, sms = 0, smem_optin = 0;
  if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device) != cudaSuccess || major != 10) return false;
  if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) return false;
  if (cudaDeviceGetAttribute(&smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, device) != cudaSuccess) return false;
  if ((size_t)smem_optin < smem_bytes(d, false) || (size_t)smem_optin < smem_bytes(d, true)) return false;
  return d.H / kUnits * d.ndir <= sms;
}

cudaError_t gru_persistent_forward(const GruDims& d, const float* w_hh, const float* b_hh, const float* gx, float* y, float* rsv,
                                   uint32_t* sync, uint32_t* status, double timeout_s, cudaStream_t stream) {
  if (!dims_ok(d) || !aligned16(w_hh) || !aligned16(y)) return cudaErrorInvalidValue;
  CUtensorMap tm_w, tm_x;
  if (!make_map(&tm_w, w_hh, (uint64_t)d.ndir * 3 * d.H, (uint64_t)d.H, kUnits)) return cudaErrorInvalidValue;
  if (!make_map(&tm_x, y, (uint64_t)d.T * d.B, (uint64_t)d.ndir * d.H, kBatchTile)) return cudaErrorInvalidValue;
  Params p{};
  p.d = d;
  p.b_hh = b_hh;
  p.gx = gx;
  p.y = y;
  p.rsv = rsv;
  p.sync = sync;
  p.status = status;
  p.timeout_ns = (unsigned long long)(timeout_s * 1e9);
  p.prof = g_prof;
  p.debug = g_debug;
  return launch<false>(d, tm_w, tm_x, p, stream);
}

cudaError_t gru_persistent_backward(const GruDims& d, const float* w_hh_t, const float* y, const float* rsv, const float* dy,
                                    float* dgx, float* dgh, uint32_t* sync, uint32_t* status, double timeout_s,
                                    cudaStream_t stream) {
  if (!dims_ok(d) || !aligned16(w_hh_t) || !aligned16(dgh)) return cudaErrorInvalidValue;
  CUtensorMap tm_w, tm_x;
  if (!make_map(&tm_w, w_hh_t, (uint64_t)d.ndir * d.H, (uint64_t)3 * d.H, kUnits)) return cudaErrorInvalidValue;
  if (!make_map(&tm_x, dgh, (uint64_t)d.T * d.B, (uint64_t)d.ndir * 3 * d.H, kBatchTile)) return cudaErrorInvalidValue;
  Params p{};
  p.d = d;
  p.y = const_cast<float*>(y);
  p.rsv = const_cast<float*>(rsv);
  p.dy = dy;
  p.dgx = dgx;
  p.dgh = dgh;
  p.sync = sync;
  p.status = status;
  p.timeout_ns = (unsigned long long)(timeout_s * 1e9);
  p.prof = g_prof;
  p.debug = g_debug;
  return launch<true>(d, tm_w, tm_x, p, stream);
}

}  // namespace gpu
}  // namespace bc
