// Persistent bidirectional GRU layer for sm_100a (see gru_persistent.h for the interface).
//
// Work split. Direction d of a layer is run by H/16 blocks (grid.y = direction); block c owns
// the hidden units [16c, 16c+16) and produces their outputs. For the recurrent product the blocks
// work in groups of C (4 forward, 16 backward at H = 1024) that split the reduction length K among
// themselves: block q of a group keeps, for ALL units of its group, the weight columns of its K
// range in shared memory for the whole sequence (forward 48C rows x H/C columns, backward 16C
// rows x 3H/C columns: 192 KiB of fp32 at H = 1024 either way). Each time step it
//   1. waits until every block of its direction has published the operand of this step (h_{t-1}
//      forward, the pre-activation gradients backward; a counter in global memory,
//      release/acquire at gpu scope, bounded wait),
//   2. brings its K range of that operand (32 batch rows x K/C) into shared memory with TMA
//      (cp.async.bulk.tensor, 128-byte swizzle) while one thread issues tcgen05.mma (TF32
//      operands, M = 64 accumulator rows of which 32 are the batch, N = the group's weight rows,
//      K = 8 per instruction) into an accumulator in tensor memory,
//   3. reads the accumulator back (tcgen05.ld), sends every other member of the group the partial
//      sums of that member's units through global memory, meets the group (a second counter),
//      adds up the C partial sums of its own units,
//   4. applies the gate non-linearities (forward) or forms the next pre-activation gradients
//      (backward) for its 16 units, writes the results and signals the direction's counter.
// Why the split: one tcgen05.mma costs about 55-60 ns here almost regardless of its shape
// (measured: M x N = 128 x 32, 64 x 32 and 64 x 192 all take the same time), and a step needs K/8
// of them in a row. Splitting K over C blocks divides that chain by C; the price is the exchange
// of C - 1 small partial-sum tiles per step.
//
// The MMA reads 64 operand rows starting at a tile's base while a tile of the streamed operand
// has 32; the rest aliases what follows in shared memory (the next tile, finally the weight
// area) and only produces accumulator rows that are never read.
//
// Every wait (mbarrier, step counter) is bounded by %globaltimer. When a wait runs out the block
// records a status bit, waits (bounded) for its own copies and MMAs in flight, frees its tensor
// memory and returns.
#include "gru_persistent.h"

#include <cuda.h>

#include <algorithm>
#include <atomic>
#include <mutex>

namespace bc {
namespace gpu {

namespace {

constexpr int kUnits = 16;            // hidden units per block
constexpr int kBatchTile = 32;        // batch entries: rows of one TMA box of the streamed operand, the valid rows of the MMA's M
constexpr int kKTile = 32;            // fp32 elements in one 128-byte swizzle row
constexpr int kTilesPerStage = 4;     // K tiles per pipeline stage (K = 128)
constexpr int kStageBytes = kTilesPerStage * kBatchTile * 128;   // 16 KiB
constexpr int kXTileBytes = kBatchTile * 128;                    // 4 KiB
constexpr int kComputeThreads = 128;   // four warps: accumulator read-back, exchange, gate math
constexpr int kThreads = 160;          // plus one warp whose first thread issues copies and MMAs
constexpr int kMaxBlocksPerDir = 64;   // H / 16 at H = 1024
constexpr int kMmaM = 64;            // smallest M of tcgen05.mma; the batch fills 32 of its rows (an MMA costs the same for M = 128)

struct Params {
  GruDims d;
  const float* b_hh;    // forward
  const float* gx;      // forward
  float* y;             // forward: out; backward: in (const)
  float* rsv;           // forward: out; backward: in
  const float* dy;      // backward
  float* dgx;           // backward
  float* dgh;           // backward
  float* xchg;          // partial sums exchanged inside a group
  int split;            // blocks per group: each holds 1/split of the reduction length
  uint32_t* sync;
  uint32_t* status;
  unsigned long long timeout_ns;
  unsigned long long* prof;   // optional: 8 time stamps per step of block (0, 0), for tuning
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
// 32 consecutive accumulator columns of this thread's TMEM lane; tc_ld_wait() before the values are used,
// so that several loads can be in flight.
__device__ __forceinline__ void tc_ld32_issue(uint32_t taddr, float* v) {
  uint32_t* r = reinterpret_cast<uint32_t*>(v);
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
        "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
        "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tc_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

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

// One recurrent product of this block: wait until the peers have published the operand of this
// step, stream the block's K range of it (32 rows x kq columns) through the two stages with TMA,
// and accumulate D[batch, n] += X[batch, k] * W[n, k] in tensor memory (M = 64 rows of which the
// first 32 are the batch, N = the group's weight rows). Thread 0 only.
//   row0 / col0: first row and first column of the block's operand part in the tensor map
//   ntiles: K tiles (32 columns each) of the block's K range
__device__ __forceinline__ uint32_t drive_product(Driver& dr, const CUtensorMap* tm_x, int row0, int col0, int ntiles, uint32_t w_addr,
                                                  int w_tile_bytes, uint32_t x_addr, uint32_t bars, uint32_t tmem, uint32_t idesc,
                                                  const uint32_t* ctr, uint32_t target, unsigned long long timeout_ns,
                                                  unsigned long long* stamp) {
  const uint32_t full0 = bars, empty0 = bars + 16, done = bars + 32;
  if (!wait_counter(ctr, target, timeout_ns)) return kGruTimeoutGrid;
  if (stamp) stamp[1] = gtimer();
  fence_proxy_async();   // peers wrote the operand with ordinary stores; TMA reads it through the async proxy
  const int nstages = (ntiles + kTilesPerStage - 1) / kTilesPerStage;
  auto load_stage = [&](int sg) {
    const int st = sg & 1, t0 = sg * kTilesPerStage, nt = min(kTilesPerStage, ntiles - t0);
    mbar_expect_tx(full0 + 8 * st, (uint32_t)(nt * kXTileBytes));
    dr.pending[st] = true;
    for (int i = 0; i < nt; i++)
      tma_load_2d(x_addr + st * kStageBytes + i * kXTileBytes, tm_x, col0 + (t0 + i) * kKTile, row0, full0 + 8 * st);
  };
  load_stage(0);
  if (nstages > 1) load_stage(1);
  // Descriptors differ from tile to tile only in their address field (bits 0-13, units of 16
  // bytes), which cannot carry into the next field: all addresses lie below 256 KiB.
  const uint64_t a_desc0 = operand_desc(x_addr), b_desc0 = operand_desc(w_addr);
  for (int sg = 0; sg < nstages; sg++) {
    const int st = sg & 1, t0 = sg * kTilesPerStage, nt = min(kTilesPerStage, ntiles - t0);
    if (!mbar_wait(full0 + 8 * st, dr.full_phase[st], timeout_ns, nullptr)) return kGruTimeoutCopy;
    dr.full_phase[st] ^= 1;
    dr.pending[st] = false;
    if (stamp && sg == 0) stamp[2] = gtimer();
    tc_fence_after();
    for (int i = 0; i < nt; i++) {
      const uint64_t a_i = a_desc0 + (uint64_t)((st * kStageBytes + i * kXTileBytes) >> 4);
      const uint64_t b_i = b_desc0 + (uint64_t)(((uint32_t)(t0 + i) * (uint32_t)w_tile_bytes) >> 4);
      if (t0 + i == 0) {
        tc_mma_tf32(tmem, a_i, b_i, idesc, 0u);
#pragma unroll
        for (int ks = 1; ks < 4; ks++) tc_mma_tf32_acc(tmem, a_i + 2 * ks, b_i + 2 * ks, idesc);
      } else {
#pragma unroll
        for (int ks = 0; ks < 4; ks++) tc_mma_tf32_acc(tmem, a_i + 2 * ks, b_i + 2 * ks, idesc);
      }
    }
    if (sg + 2 < nstages) {
      // Longer K ranges than two stages: refill this stage as soon as its MMAs have read it.
      tc_commit(empty0 + 8 * st);
      if (!mbar_wait(empty0 + 8 * st, dr.empty_phase[st], timeout_ns, nullptr)) return kGruTimeoutMma;
      dr.empty_phase[st] ^= 1;
      load_stage(sg + 2);
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
  const bool driver = tid == kComputeThreads;   // does nothing but wait for peers, issue TMA copies and MMAs
  const int dir = blockIdx.y, u0 = blockIdx.x * kUnits;
  const int T = p.d.T, B = p.d.B, H = p.d.H, ND = p.d.ndir;
  const int nblocks = gridDim.x;
  constexpr int kRows = BWD ? kUnits : 3 * kUnits;     // weight rows per owner: its units (x 3 gates forward)
  const int C = p.split;                               // blocks per group = K split
  const int grp = blockIdx.x / C, q = blockIdx.x % C;  // group and this block's K range / member index
  const int kdim = BWD ? 3 * H : H;
  const int kq = kdim / C;                             // this block's K range is [q * kq, (q + 1) * kq)
  const int ntiles = kq / kKTile;
  const int nrows = kRows * C;                         // MMA N: weight rows of the whole group
  const int w_tile = nrows * 128;

  // Stages first: the MMA reads 64 operand rows from a 32-row tile, and what follows the last
  // tile must still be inside the allocation (it is the weight area).
  uint8_t* x_s = smem;
  uint8_t* w_s = smem + 2 * kStageBytes;
  uint64_t* bar_s = reinterpret_cast<uint64_t*>(w_s + (size_t)ntiles * w_tile);   // full[2], -, -, done, weights
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_s + 6);
  volatile int* abort_s = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const uint32_t bars = smem_u32(bar_s);
  const uint32_t done_bar = bars + 32, w_bar = bars + 40;
  const uint32_t tmem_cols = nrows <= 32 ? 32u : nrows <= 64 ? 64u : nrows <= 128 ? 128u : 256u;

  if (tid == 0) {
    for (int i = 0; i < 6; i++) mbar_init(bars + 8 * i, 1);
    *abort_s = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(tmem_cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  // The group's weight rows for this block's K range: loaded once, resident for the whole
  // sequence. Row order inside a tile: owner (member of the group), then gate, then unit.
  if (driver) {
    mbar_expect_tx(w_bar, (uint32_t)(ntiles * w_tile));
    for (int kt = 0; kt < ntiles; kt++) {
      for (int m = 0; m < C; m++) {
        const int unit0 = (grp * C + m) * kUnits;
        if (BWD) {
          tma_load_2d(smem_u32(w_s) + kt * w_tile + m * (kUnits * 128), &tm_w, q * kq + kt * kKTile, dir * H + unit0, w_bar);
        } else {
          for (int g = 0; g < 3; g++)
            tma_load_2d(smem_u32(w_s) + kt * w_tile + (m * 3 + g) * (kUnits * 128), &tm_w, q * kq + kt * kKTile,
                        dir * 3 * H + g * H + unit0, w_bar);
        }
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
  const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(nrows >> 3) << 17) | ((uint32_t)(kMmaM >> 4) << 24);

  // Compute thread (u, bq) handles unit u0 + u for the batch entries bq, bq + 8, bq + 16, bq + 24.
  // The driver's warp gets bq = 32, which fails every `b < B` test below.
  const int u = tid & 15, bq = tid < kComputeThreads ? tid >> 4 : 32;
  float carry[4] = {0.f, 0.f, 0.f, 0.f};   // forward: h_{t-1}; backward: recurrent part of dh_t
  float bias_r = 0.f, bias_z = 0.f, bias_n = 0.f;
  if (!BWD) {
    bias_r = p.b_hh[dir * 3 * H + u0 + u];
    bias_z = p.b_hh[dir * 3 * H + H + u0 + u];
    bias_n = p.b_hh[dir * 3 * H + 2 * H + u0 + u];
  }
  uint32_t* dir_ctr = p.sync + dir;                                 // one arrival per block and published step
  // Partial sums travel through global memory: xchg[dir][group][owner][source][batch 32][kRows].
  // A tile is rewritten only after the direction's step barrier, which every reader passes after
  // it has consumed the previous contents.
  float* xg = p.xchg + ((size_t)(dir * (nblocks / C) + grp) * C) * C * (32 * kRows);
  uint32_t* grp_ctr = p.sync + 8 + dir * kMaxBlocksPerDir + grp;   // one arrival per member and product
  BwdInputs pre;
  uint32_t products = 0;
  constexpr int kMaxC = BWD ? 16 : 4;
  // The block's whole accumulator in shared memory, one row of nrows floats per batch entry (it
  // aliases the stages between products). 16-byte slot n/4 of row b sits at slot (n/4) ^ (b & swz),
  // so that the 16 threads that write one slot of 16 different rows at a time hit all banks.
  float* t_s = reinterpret_cast<float*>(x_s);
  float4* t4 = reinterpret_cast<float4*>(x_s);
  const int row4 = nrows / 4;                          // 16-byte slots per row
  const int swz = (nrows % 32 == 0) ? 7 : 0;
  constexpr int kRows4 = kRows / 4;

  // Exchange after a product. (1) The accumulator goes to shared memory: rows 16w .. 16w+15 of the
  // M = 64 accumulator live in lanes 0-15 of the TMEM quarter that warp w may read, so threads
  // (w < 2, lane < 16) hold batch entry 16w + lane and write 32 consecutive columns as eight
  // 16-byte stores. (2) Every member's columns are copied, as a [32][kRows] tile, to that member's
  // place in global memory with coalesced 16-byte stores. (3) The group meets (one release,
  // counter). (4) The block adds the tiles it received to its own columns, in place.
  // Returns false if the group did not arrive in time.
  auto exchange = [&]() {
    if (warp < 2) {
      const int b = warp * 16 + lane;
      // Two loads in flight. Columns past nrows that a load touches are still inside the
      // allocation (nrows rounded up to a power of two, at least 32) and are not stored.
      for (int c0 = 0; c0 < nrows; c0 += 64) {
        float v[32], w[32];
        const bool two = c0 + 32 < nrows;
        tc_ld32_issue(tmem + ((uint32_t)(warp * 32) << 16) + (uint32_t)c0, v);
        if (two) tc_ld32_issue(tmem + ((uint32_t)(warp * 32) << 16) + (uint32_t)(c0 + 32), w);
        tc_ld_wait();
        if (lane < 16) {
          float4* row = t4 + b * row4;
#pragma unroll
          for (int k = 0; k < 8; k++)
            if (c0 + 4 * k < nrows) row[((c0 >> 2) + k) ^ (b & swz)] = make_float4(v[4 * k], v[4 * k + 1], v[4 * k + 2], v[4 * k + 3]);
          if (two) {
#pragma unroll
            for (int k = 0; k < 8; k++)
              if (c0 + 32 + 4 * k < nrows) row[((c0 >> 2) + 8 + k) ^ (b & swz)] = make_float4(w[4 * k], w[4 * k + 1], w[4 * k + 2], w[4 * k + 3]);
          }
        }
      }
    }
    tc_fence_before();
    __syncthreads();
    constexpr int kTile4 = 32 * kRows4;                // 16-byte words of one member's tile
    for (int idx = tid; idx < C * kTile4; idx += kThreads) {
      const int owner = idx / kTile4, w4 = idx - owner * kTile4;
      if (owner != q) {
        const int b = w4 / kRows4, j4 = w4 - b * kRows4;
        __stcg(reinterpret_cast<float4*>(xg + (size_t)(owner * C + q) * (32 * kRows)) + w4, t4[b * row4 + ((owner * kRows4 + j4) ^ (b & swz))]);
      }
    }
    products += 1;
    bool good = true;
    if (C > 1) {
      // The barrier orders every thread's stores before thread 0's release (cumulativity), so one
      // release at gpu scope publishes the whole tile.
      __syncthreads();
      if (tid == 0) {
        signal_counter(grp_ctr);
        good = wait_counter(grp_ctr, (uint32_t)C * products, p.timeout_ns);
        if (!good) { atomicOr(p.status, kGruTimeoutGrid); *abort_s = 1; }
      }
      good = __syncthreads_and(good) != 0;
    }
    if (good) {
      for (int w4 = tid; w4 < kTile4; w4 += kThreads) {
        float4 part[kMaxC];
#pragma unroll
        for (int m = 0; m < kMaxC; m++) {
          part[m] = make_float4(0.f, 0.f, 0.f, 0.f);
          if (m < C && m != q) part[m] = __ldcg(reinterpret_cast<const float4*>(xg + (size_t)(q * C + m) * (32 * kRows)) + w4);
        }
        const int b = w4 / kRows4, j4 = w4 - b * kRows4;
        float4* own = t4 + b * row4 + ((q * kRows4 + j4) ^ (b & swz));
        float4 acc = *own;
#pragma unroll
        for (int m = 0; m < kMaxC; m++) { acc.x += part[m].x; acc.y += part[m].y; acc.z += part[m].z; acc.w += part[m].w; }
        *own = acc;
      }
    }
    __syncthreads();
    return good;
  };
  // Summed pre-activation (forward: gate g) of unit u0 + u for batch entry b, after exchange().
  auto summed = [&](int g, int b) {
    const int n = q * kRows + g * kUnits + u;
    return t_s[(b * row4 + ((n >> 2) ^ (b & swz))) * 4 + (n & 3)];
  };

  for (int s = 0; ok && s < T; s++) {
    uint32_t fail = 0;
    unsigned long long* stamp = (p.prof && (tid == 0 || driver) && blockIdx.x == 0 && blockIdx.y == 0) ? p.prof + (size_t)s * 8 : nullptr;
    if (stamp && tid == 0) stamp[0] = gtimer();
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
        if (driver) {
          fail = drive_product(dr, &tm_x, tprev * B, dir * H + q * kq, ntiles, smem_u32(w_s), w_tile, smem_u32(x_s), bars, tmem, idesc,
                               dir_ctr, (uint32_t)nblocks * (uint32_t)s, p.timeout_ns, stamp);
          if (fail) { atomicOr(p.status, fail); *abort_s = 1; }
        }
        __syncwarp();
        bool got = mbar_wait(done_bar, done_phase, 4 * p.timeout_ns, abort_s);
        got = __all_sync(0xffffffffu, got) != 0;
        if (got) done_phase ^= 1;
        if (stamp && tid == 0) stamp[4] = gtimer();
        tc_fence_after();
        if (!got || fail) tc_fence_before();
        ok = __syncthreads_and(got && !fail) != 0;
        if (!ok) { mma_in_flight = true; break; }
        ok = exchange();
        if (!ok) break;
      }
      float rsv_r[4], rsv_z[4], rsv_n[4], rsv_hn[4];
#pragma unroll
      for (int j = 0; j < 4; j++) {
        const int b = bq + 8 * j;
        if (b < B) {
          float hr = bias_r, hz = bias_z, hn = bias_n;
          if (s > 0) {
            hr += summed(0, b);
            hz += summed(1, b);
            hn += summed(2, b);
          }
          const float r = sigmoidf_(gxr[j] + hr);
          const float z = sigmoidf_(gxz[j] + hz);
          const float n = tanhf(gxn[j] + r * hn);
          const float h = n + z * (carry[j] - n);
          carry[j] = h;
          p.y[((size_t)t * B + b) * (ND * H) + dir * H + u0 + u] = h;
          rsv_r[j] = r; rsv_z[j] = z; rsv_n[j] = n; rsv_hn[j] = hn;
        }
      }
      if (stamp && tid == 0) stamp[5] = gtimer();
      if (s + 1 < T) {
        fence_proxy_async();   // the peers read these stores through TMA
        __syncthreads();
        if (tid == 0) signal_counter(dir_ctr);   // release at gpu scope, cumulative over the barrier
      }
      if (stamp && tid == 0) stamp[6] = gtimer();
      // The saved activations are not needed by the peers: written after the step is published.
#pragma unroll
      for (int j = 0; j < 4; j++) {
        const int b = bq + 8 * j;
        if (b < B) {
          float* rs = p.rsv + (((size_t)(dir * T + t) * B + b) * 4) * H + u0 + u;
          rs[0] = rsv_r[j]; rs[H] = rsv_z[j]; rs[2 * H] = rsv_n[j]; rs[3 * H] = rsv_hn[j];
        }
      }
    } else {
      // ---------------- backward step ----------------
      const int t = dir ? s : T - 1 - s;
      if (s == 0) load_bwd_inputs(p, pre, t, dir, u0 + u, bq);
      float keep[4], g_r[4], g_z[4], g_n[4];
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
          p.dgh[o] = drr; p.dgh[o + H] = dz; p.dgh[o + 2 * H] = dn * r;
          g_r[j] = drr; g_z[j] = dz; g_n[j] = dn;
          keep[j] = dh * z;
        }
      }
      if (stamp && tid == 0) stamp[5] = gtimer();
      if (s + 1 < T) {
        fence_proxy_async();   // the peers read these stores through TMA
        __syncthreads();
        if (tid == 0) signal_counter(dir_ctr);   // release at gpu scope, cumulative over the barrier
      }
      if (stamp && tid == 0) stamp[6] = gtimer();
      // dgx is only read after the kernel: written after the step is published.
#pragma unroll
      for (int j = 0; j < 4; j++) {
        const int b = bq + 8 * j;
        if (b < B) {
          const size_t o = (((size_t)t * B + b) * ND + dir) * 3 * H + u0 + u;
          p.dgx[o] = g_r[j]; p.dgx[o + H] = g_z[j]; p.dgx[o + 2 * H] = g_n[j];
        }
      }
      if (s + 1 < T) {
        // Next step's saved activations and output gradient: in flight while the product runs.
        load_bwd_inputs(p, pre, dir ? s + 1 : T - 2 - s, dir, u0 + u, bq);
        if (driver) {
          fail = drive_product(dr, &tm_x, t * B, dir * 3 * H + q * kq, ntiles, smem_u32(w_s), w_tile, smem_u32(x_s), bars, tmem, idesc,
                               dir_ctr, (uint32_t)nblocks * (uint32_t)(s + 1), p.timeout_ns, stamp);
          if (fail) { atomicOr(p.status, fail); *abort_s = 1; }
        }
        __syncwarp();
        bool got = mbar_wait(done_bar, done_phase, 4 * p.timeout_ns, abort_s);
        got = __all_sync(0xffffffffu, got) != 0;
        if (got) done_phase ^= 1;
        if (stamp && tid == 0) stamp[4] = gtimer();
        tc_fence_after();
        if (!got || fail) tc_fence_before();
        ok = __syncthreads_and(got && !fail) != 0;
        if (!ok) { mma_in_flight = true; break; }
        ok = exchange();
        if (!ok) break;
#pragma unroll
        for (int j = 0; j < 4; j++) {
          const int b = bq + 8 * j;
          carry[j] = b < B ? keep[j] + summed(0, b) : 0.f;
        }
        __syncthreads();   // the summed tile lives in the stage area, which the next product's first copy overwrites
      }
    }
  }

  // Leave cleanly: nothing of this block may still be in flight when tensor memory is freed.
  if (driver && (mma_in_flight || !ok)) {
    for (int st = 0; st < 2; st++)
      if (dr.pending[st]) mbar_wait(bars + 8 * st, dr.full_phase[st], p.timeout_ns, nullptr);
    tc_commit(done_bar);
    mbar_wait(done_bar, done_phase, p.timeout_ns, nullptr);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    __syncwarp();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(tmem_cols) : "memory");
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

size_t smem_bytes(const GruDims& d, bool bwd) {
  const size_t kdim = bwd ? 3 * (size_t)d.H : (size_t)d.H;
  const size_t rows = bwd ? kUnits : 3 * kUnits;
  return (kdim / kKTile) * rows * 128 + 2 * kStageBytes + 128 + 1024;
}

bool dims_ok(const GruDims& d) {
  return d.T >= 1 && d.T < 4096 && d.B >= 1 && d.B <= kBatchTile && d.H >= 128 && d.H <= 1024 && d.H % 128 == 0 && (d.ndir == 1 || d.ndir == 2);
}

bool aligned16(const void* p) { return ((uintptr_t)p & 15) == 0; }

// Blocks per group (= K split): the largest supported value for which the group's weight rows fit
// one MMA (N <= 256), every block gets whole K tiles, and groups tile the direction's blocks.
int choose_split(const GruDims& d, bool bwd) {
  const int blocks = d.H / kUnits, kdim = bwd ? 3 * d.H : d.H, rows = bwd ? kUnits : 3 * kUnits;
  for (int c : {16, 8, 4, 2, 1}) {
    if (c > (bwd ? 16 : 4)) continue;
    if (rows * c > 256 || blocks % c != 0 || kdim % (c * kKTile) != 0) continue;
    return c;
  }
  return 1;
}

size_t xchg_floats(const GruDims& d, bool bwd) {
  const size_t rows = bwd ? kUnits : 3 * kUnits;
  return (size_t)d.ndir * (d.H / kUnits) * choose_split(d, bwd) * 32 * rows;
}

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
  if (grid.x > (unsigned)kMaxBlocksPerDir) return cudaErrorInvalidValue;
  if ((int)(grid.x * grid.y) > per_sm * sms) return cudaErrorCooperativeLaunchTooLarge;
  void* args[] = {(void*)&tm_w, (void*)&tm_x, (void*)&p};
  return cudaLaunchCooperativeKernel((const void*)kernel, grid, block, args, smem, stream);
}

}  // namespace

void gru_persistent_set_profile(unsigned long long* stamps) { g_prof = stamps; }

bool gru_persistent_supported(const GruDims& d, int device) {
  if (!dims_ok(d) || !encode_fn()) return false;
  int major = 0, sms = 0, smem_optin = 0;
  if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device) != cudaSuccess || major != 10) return false;
  if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) return false;
  if (cudaDeviceGetAttribute(&smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, device) != cudaSuccess) return false;
  if ((size_t)smem_optin < smem_bytes(d, false) || (size_t)smem_optin < smem_bytes(d, true)) return false;
  return d.H / kUnits * d.ndir <= sms;
}

size_t gru_persistent_workspace_bytes(const GruDims& d) {
  if (!dims_ok(d)) return 0;
  return std::max(xchg_floats(d, false), xchg_floats(d, true)) * sizeof(float);
}

cudaError_t gru_persistent_forward(const GruDims& d, const float* w_hh, const float* b_hh, const float* gx, float* y, float* rsv,
                                   float* workspace, uint32_t* sync, uint32_t* status, double timeout_s, cudaStream_t stream) {
  if (!dims_ok(d) || !aligned16(w_hh) || !aligned16(y) || !aligned16(workspace)) return cudaErrorInvalidValue;
  CUtensorMap tm_w, tm_x;
  if (!make_map(&tm_w, w_hh, (uint64_t)d.ndir * 3 * d.H, (uint64_t)d.H, kUnits)) return cudaErrorInvalidValue;
  if (!make_map(&tm_x, y, (uint64_t)d.T * d.B, (uint64_t)d.ndir * d.H, kBatchTile)) return cudaErrorInvalidValue;
  Params p{};
  p.d = d;
  p.b_hh = b_hh;
  p.gx = gx;
  p.y = y;
  p.rsv = rsv;
  p.xchg = workspace;
  p.split = choose_split(d, false);
  p.sync = sync;
  p.status = status;
  p.timeout_ns = (unsigned long long)(timeout_s * 1e9);
  p.prof = g_prof;
  return launch<false>(d, tm_w, tm_x, p, stream);
}

cudaError_t gru_persistent_backward(const GruDims& d, const float* w_hh_t, const float* y, const float* rsv, const float* dy,
                                    float* dgx, float* dgh, float* workspace, uint32_t* sync, uint32_t* status, double timeout_s,
                                    cudaStream_t stream) {
  if (!dims_ok(d) || !aligned16(w_hh_t) || !aligned16(dgh) || !aligned16(workspace)) return cudaErrorInvalidValue;
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
  p.xchg = workspace;
  p.split = choose_split(d, true);
  p.sync = sync;
  p.status = status;
  p.timeout_ns = (unsigned long long)(timeout_s * 1e9);
  p.prof = g_prof;
  return launch<true>(d, tm_w, tm_x, p, stream);
}

}  // namespace gpu
}  // namespace bc
