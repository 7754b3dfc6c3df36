// Host-visible launch interface of the peer-memory collective kernels.
//
// One launch = one collective on one rank. The same kernels also run "emulated": a single
// cooperative launch whose blockIdx.y selects one of several ranks whose buffers all live on one
// GPU. That is how the multi-rank protocol is tested on a single device, where separate launches
// that wait on one another must never be used.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "../common.h"
#include "layout.h"

namespace bc {
namespace gpu {

enum class Algo : int { AUTO = 0, ONE_SHOT = 1, TWO_SHOT = 2, NVLS = 3 };
inline const char* algo_name(Algo a) {
  switch (a) {
    case Algo::AUTO: return "auto";
    case Algo::ONE_SHOT: return "one_shot";
    case Algo::TWO_SHOT: return "two_shot";
    case Algo::NVLS: return "nvls";
  }
  return "?";
}

enum class OptKind : int { NONE = 0, SGD = 1, ADAM = 2 };

// Optimizer update fused behind the reduction. Formulas:
//   SGD  (TF ApplyMomentum, core/kernels/training_ops_gpu.cu.cc:82-100; torch.optim.SGD):
//        g += wd*p;  buf = first ? g : mu*buf + (1-dampening)*g;  d = nesterov ? g + mu*buf : buf;
//        p -= lr*d        (mu == 0: p -= lr*g, no buffer)
//   ADAM (TF ApplyAdam, training_ops_gpu.cu.cc:103-145, python/training/adam.py:50-60; torch AdamW):
//        decoupled: p *= 1 - lr*wd      else: g += wd*p
//        m = b1*m + (1-b1)*g;  v = b2*v + (1-b2)*g*g
//        torch form: p -= (lr/bc1) * m / (sqrt(v)/sqrt(bc2) + eps)
//        TF form   : p -= lr*sqrt(bc2)/bc1 * m / (sqrt(v) + eps)        ("epsilon hat")
// bc1 = 1 - b1^t, bc2 = 1 - b2^t are computed on the host for step t.
struct OptHyper {
  int kind;              // OptKind
  float lr;
  float weight_decay;
  float momentum;        // SGD mu
  float dampening;
  int nesterov;
  int first_step;        // SGD: momentum buffer is uninitialised (torch copies g into it)
  float beta1, beta2, eps;
  float bias_c1, bias_c2;
  int decoupled_wd;      // AdamW
  int tf_epsilon_hat;
  int zero_grad;         // write zeros over the gradient once it has been consumed
};

// Per-rank operands of a reduction launch.
struct ArRank {
  dev::RankCtx ctx;
  char* in[dev::kMaxRanks];   // every rank's input buffer as mapped here (16-byte aligned)
  char* mc_in;                // multicast mapping of the same buffer (NVLS) or null
  const char* src;            // private input that the kernel first copies into in[rank] (staged path), or null
  unsigned long long place;   // in place on symmetric memory: 1 + the offset this rank passed, compared across
                              // the ranks on the device (a mismatch sets kStatusLayout); 0 = not checked
  void* out;                  // local result; may alias in[rank]
  // fused optimizer operands (local, flat, same element order as the gradient)
  void* param;                // fp32 or same 16-bit type as the gradient
  float* master;              // fp32 master copy when param is 16-bit, else null
  float* state1;              // momentum buffer / Adam m
  float* state2;              // Adam v
};

struct ArArgs {
  int nranks_here;            // 1, or the number of emulated ranks (grid.y)
  int algo;                   // Algo (resolved, not AUTO)
  size_t count;               // elements
  float scale;                // applied to floating sums (1/size when averaging)
  int idiv;                   // integer divisor when averaging integer tensors
  int red;                    // ReduceOp; anything but SUM goes with no scale, no update and no NVLS
  int phase1_blocks;          // two-phase algorithms: 0 = every block takes part in the cross-rank phase; else only
                              // the first phase1_blocks do (NVLS wants few blocks, the local copy and update
                              // phases many) and the blocks of a rank meet at local barriers in between
  unsigned long long* prof;   // optional device array of kProfStamps: %globaltimer of block 0 of rank slot 0 at
                              // kernel entry, after barrier 1, after phase 1, after barrier 2, at the end
  OptHyper opt;
  ArRank r[dev::kMaxRanks];
};

// Per-rank operands of the staged pipeline launch (allreduce of a tensor outside symmetric
// memory in one kernel whose copier blocks and reducer blocks work on different chunks).
struct PipeRank {
  dev::RankCtx ctx;
  char* stage[dev::kMaxRanks];      // every rank's staging ring as mapped here
  char* mc_stage;                   // multicast mapping of the ring (NVLS) or null
  const char* src;                  // private input (16-byte aligned)
  char* out;                        // private output (16-byte aligned; may equal src)
  uint32_t* progress[dev::kMaxRanks];  // progress[p] = the progress words inside rank p's pad: [2][kPipeMaxGroups][kMaxRanks]
  uint32_t* local;                  // this rank's arrival counters, zeroed before the launch: [2][nchunks]
};

struct PipeArgs {
  int nranks_here;            // 1, or the number of emulated ranks (grid.y)
  size_t npacks;              // 16-byte packs to reduce
  size_t chunk_packs;         // packs per chunk (the last chunk may be shorter)
  int nchunks;
  int slots;                  // chunks that the staging ring holds
  int lag;                    // chunks by which the copy-out trails the copy-in (< slots unless everything fits;
                              // a multiple of cgroups)
  int reducers;               // the first `reducers` blocks of a rank reduce, the others copy
  int rgroups, cgroups;       // groups of reducer / copier blocks; group g takes the chunks c with c % groups == g
  int streaming;              // reducer blocks never drain between chunks: 15 warps move data, one warp watches
                              // the progress words and publishes finished chunks
  uint32_t base;              // value of the progress words before this launch (a launch adds at most
                              // ceil(nchunks / groups) to a word)
  float scale;
  int idiv;
  PipeRank r[dev::kMaxRanks];
};

// Per-rank operands of a variable-length allgather launch.
struct AgRank {
  dev::RankCtx ctx;
  const char* in;             // local slab
  unsigned long long bytes;   // its size
  char* base[dev::kMaxRanks]; // every rank's output segment base as mapped here
  char* mc_base;              // multicast mapping of the same segment (NVLS), or null: P2P stores only
  unsigned long long out_off; // where this rank's output starts inside its own segment
  unsigned long long* sizes_out;  // optional local array [world]: every rank's slab size in bytes
  unsigned long long capacity;    // bytes available from every rank's segment base (0 = unknown); bounds-checked builds only
};

struct AgArgs {
  int nranks_here;
  AgRank r[dev::kMaxRanks];
};

constexpr int kProfStamps = 5;

struct LaunchCfg {
  int blocks = 0;     // 0 = choose from size
  int threads = 512;
  bool cooperative = false;   // required when nranks_here > 1
};

// Launch the reduction. `param_dtype` is F32, or equal to `dtype` for 16-bit parameters.
cudaError_t launch_allreduce(const ArArgs& a, DType dtype, DType param_dtype, const LaunchCfg& cfg, cudaStream_t s);
cudaError_t launch_allgatherv(const AgArgs& a, const LaunchCfg& cfg, cudaStream_t s);
// A streaming reducer block (544 threads: 16 warps that move data, one that waits and publishes)
// moves kPipeDataThreads x batch packs per step; a chunk whose share per rank is a multiple of
// that keeps every lane busy in every batch.
constexpr int kPipeDataThreads = 512;
constexpr int kPipeStreamingThreads = kPipeDataThreads + 32;
constexpr int kPipeSwitchBatch = 4, kPipePeerBatch = 2;
// Sum (scaled) of private tensors through the staging rings; `nvls` needs a float type.
cudaError_t launch_staged_pipeline(const PipeArgs& a, DType dtype, bool nvls, const LaunchCfg& cfg, cudaStream_t s);
// Plain device copy kernel (staging of tensors that are not in symmetric memory).
cudaError_t launch_copy(void* dst, const void* src, size_t bytes, cudaStream_t s);

// Largest grid.x for which an emulated launch of `nranks` ranks is co-resident on `device`.
int max_emulated_blocks(int device, int nranks, int threads);
// Grid of a reduction launch: a pure function of its arguments, the same on every rank.
// `beside_compute`: the launch overlaps the backward pass (gradient buckets launched from
// hooks), so it is sized for the SMs that a persistent compute kernel leaves free.
int choose_blocks(size_t bytes, int world, int algo, bool fused_opt, int sm_count, int cap_override, bool beside_compute = false);

}  // namespace gpu
}  // namespace bc
