/* Public C interface of the native collectives library.
 *
 * Conventions: functions return 0 or a non-negative value on success and -1 (or NULL) on failure;
 * bc_last_error() gives the message for the calling thread. dtype codes: 0 float32, 1 int32,
 * 2 int64, 3 bfloat16, 4 float16, 5 float64, 6 uint8. device_kind: 0 host memory, 1 CUDA memory.
 * Algorithm codes: 1 one-shot, 2 two-shot, 3 NVLS (multimem).
 */
#ifndef BCOLL_H_
#define BCOLL_H_

#ifdef __cplusplus
extern "C" {
#endif

const char* bc_last_error(void);

/* Process group. `device` is a CUDA ordinal or -1 for a host-only group. Byte sizes <= 0 (or < 0
 * where 0 is meaningful) keep the defaults. `fault` is a host-side fault-injection spec or NULL. */
int bc_init(int rank, int size, int local_rank, const char* addr, int port, int device, double timeout_s,
            double device_timeout_s, long long staging_bytes, long long heap_bytes, int force_algo,
            long long one_shot_max_bytes, long long nvls_min_bytes, int use_nvls, int max_blocks, int symm_mode,
            const char* fault);
int bc_initialized(void);
int bc_shutdown(void);
int bc_rank(void);
int bc_size(void);
int bc_local_rank(void);
int bc_local_size(void);
int bc_on_gpu(void);
int bc_broken(void);
/* Hosts of a group that runs in two levels (ranks on several hosts: always for a GPU group, for a
 * CPU group when every host runs several ranks or BC_NODE_GROUPS=1), else 1; and this rank's
 * host among them. With more than
 * one host the ordered launches, the fused update and user segments of symmetric memory are
 * refused: use the negotiated collectives. */
int bc_n_nodes(void);
int bc_node_index(void);
/* The two-level allreduce on a tensor in HOST memory, with the node group's control sockets
 * standing in for the NVLink level (sum inside the host, slices over the rails, gather inside the
 * host). Collective over all ranks; must not overlap any other collective of the job. Exists to
 * check the slice arithmetic and the rails on machines without GPUs. */
/* The algorithm selector and the grid size as pure functions (no GPU, no group needed): what a
 * group of `world` ranks would use for a reduction of `bytes` bytes. Algorithms: 1 one-shot,
 * 2 two-shot, 3 NVLS; force_algo 0 = choose. Negative thresholds mean the defaults. */
int bc_select_algo(int world, long long bytes, int dtype, int in_place_or_fused, int has_multicast, int force_algo,
                   long long one_shot_max_bytes, long long nvls_min_bytes, int use_nvls);
int bc_choose_blocks(long long bytes, int world, int algo, int fused_update, int sm_count, int cap_override, int beside_compute);
/* How the staged pipeline kernel cuts a tensor (pure function): out4 = chunk bytes, chunks of
 * one launch, ring slots, lag of the copy-out. chunk_bytes / slots / cgroups <= 0: the defaults;
 * unit_bytes > 0: chunks are multiples of it instead of 4 KiB. */
int bc_plan_pipeline(long long bytes, long long slice_bytes, long long chunk_bytes, int slots, int cgroups, long long unit_bytes,
                     long long* out4);
/* How a gathered result larger than the staging area is cut into rounds (pure function): returns
 * the number of rounds and writes every rank's piece size per round. */
long long bc_plan_gather_rounds(int world, const unsigned long long* all_bytes, long long staging_bytes, unsigned long long* pieces_out);
int bc_two_level_allreduce_host(void* data, long long count, int dtype, int average, int reduce_op);

/* Negotiated, name-keyed collectives. The returned handle must be released. For CUDA tensors
 * `ready_event` (a cudaEvent_t or NULL) is what the private stream waits on before touching the
 * input, and bc_done_event() is what the consumer's stream must wait on after bc_wait(). */
typedef void* (*bc_alloc_fn)(long long handle, long long total_rows, void* user, int* is_symmetric);
long long bc_allreduce_async(const char* name, const void* in, void* out, int dtype, int ndim, const long long* shape,
                             int device_kind, int average, int zero_copy, void* ready_event, int reduce_op);
/* reduce_op: 0 sum, 1 prod, 2 min, 3 max (averaging goes with the sum only). */
long long bc_allgather_async(const char* name, const void* in, int dtype, int ndim, const long long* shape, int device_kind,
                             bc_alloc_fn alloc, void* user, void* ready_event);
int bc_wait(long long handle, double timeout_s);
int bc_poll(long long handle);
void* bc_done_event(long long handle);
int bc_result_algo(long long handle);
int bc_result_dim0(long long handle, long long* out, int n);
int bc_release(long long handle);
/* Host allgather of one small blob per rank; `out` receives them back to back, `lens[r]` their sizes. */
int bc_blob_gather(const char* name, const void* data, int len, void* out, long long out_cap, int* lens);

int bc_set_fault(const char* spec);
const char* bc_stats_json(void);
int bc_clear_stats(void);
unsigned bc_device_status(void);
int bc_set_device_timeout(double seconds);

/* Symmetric memory (CUDA groups only). */
void* bc_symm_heap(long long* bytes);
void* bc_symm_new_segment(long long bytes, int* seg_id, int* has_multicast); /* collective */
int bc_symm_contains(const void* p, long long bytes);
const char* bc_symm_describe(void);
void* bc_comm_stream(int channel);
/* cudaStreamWaitEvent(stream, event) for raw handles (e.g. a torch stream and bc_done_event()). */
int bc_stream_wait_event(void* stream, void* event);

/* Optimizer update fused behind a gradient reduction; mirrors bc::gpu::OptHyper. */
typedef struct bc_opt_hyper {
  int kind; /* 1 SGD, 2 Adam */
  float lr, weight_decay, momentum, dampening;
  int nesterov, first_step;
  float beta1, beta2, eps, bias_c1, bias_c2;
  int decoupled_wd, tf_epsilon_hat, zero_grad;
} bc_opt_hyper;

/* Ordered launches on a channel's private stream, without negotiation: every rank must issue the
 * same sequence of calls per channel. `wait_event` / `record_event` are cudaEvent_t or NULL. */
int bc_allreduce_direct(int channel, const void* in, void* out, long long count, int dtype, int average,
                        void* wait_event, void* record_event);
/* `beside_compute` != 0: the launch overlaps the backward pass; its grid is capped to the SMs that a
 * persistent compute kernel leaves free (option "overlap_blocks"), so all its blocks can be resident. */
int bc_fused_step(int channel, void* grad, long long count, int dtype, void* param, float* master, float* s1, float* s2,
                  const bc_opt_hyper* h, float scale, void* wait_event, void* record_event, int beside_compute);
/* Run-time switches: "device_timing" (1: ordered launches and negotiated GPU allreduces are bracketed
 * by timing events and their records in bc_stats_json() carry "device_us"), "overlap_blocks". */
int bc_set_option(const char* key, long long value);
/* Tuning aid: device array of 5 uint64 that block 0 of later reduction launches fills with %globaltimer
 * at kernel entry, after the first barrier, after phase 1, after the second barrier and at the end
 * (one-shot: entry, barrier, reduction, end barrier, end). NULL switches it off. */
int bc_set_allreduce_profile(void* stamps);

/* Variable allgather into `out_symm`, a buffer of `capacity_bytes` (equal on all ranks) inside the
 * symmetric heap. Row counts are exchanged on the device; `sizes_out` (device memory, one entry per
 * rank, or NULL) receives every rank's slab size in bytes. */
int bc_allgatherv_direct(int channel, const void* in, long long bytes, void* out_symm, long long capacity_bytes,
                         unsigned long long* sizes_out, void* wait_event, void* record_event);

/* A group of ranks emulated on ONE GPU: each collective is a single cooperative launch. */
void* bc_emu_create(int device, int nranks, long long bytes_per_rank);
int bc_emu_destroy(void* g);
void* bc_emu_buffer(void* g, int r);
unsigned bc_emu_status(void* g);
int bc_emu_clear_status(void* g);
/* Guard regions surround every buffer and pad of the group; number of guard bytes overwritten. */
long long bc_emu_damaged_guard_bytes(void* g);
/* `srcs` (or NULL): per rank a private input that the kernel copies into the rank's buffer first (the staged
 * path). `places` (or NULL): per rank the offset it claims to reduce in place; ranks that disagree set status
 * bit 0x20000000. `prof` (or NULL): device array of 5 uint64 time stamps, see bc_set_allreduce_profile(). */
int bc_emu_allreduce(void* g, long long off, void* const* outs, long long count, int dtype, int algo, float scale, int idiv,
                     int blocks, void* stream, int reduce_op, const void* const* srcs, const unsigned long long* places, void* prof,
                     int phase1_blocks);
/* `phase1_blocks` > 0 (both calls above and below): a mixed grid, in which only that many blocks of every rank run the
 * cross-rank phase and the rank's blocks meet at two local barriers (what real groups use for NVLS launches). */
int bc_emu_fused_step(void* g, long long off, long long count, int dtype, void* const* params, float* const* masters,
                      float* const* s1, float* const* s2, const bc_opt_hyper* h, float scale, int blocks, void* stream,
                      int phase1_blocks);
/* The staged pipeline kernel (copier and reducer blocks in one launch, peer loads and stores) on
 * private tensors; the rings of `slots` chunks of `chunk_bytes` start at `off` of the buffers. */
int bc_emu_staged_pipeline(void* g, long long off, const void* const* srcs, void* const* outs, long long count, int dtype,
                           float scale, int idiv, long long chunk_bytes, int slots, int lag, int reducers, int copiers,
                           int rgroups, int cgroups, int streaming, void* stream);
int bc_emu_allgatherv(void* g, const void* const* ins, const unsigned long long* bytes, const unsigned long long* out_offs,
                      int blocks, void* stream);
int bc_emu_barrier_probe(void* g, int absent, double timeout_s, void* stream);
int bc_max_emulated_blocks(int device, int nranks);

/* Persistent bidirectional GRU layer (tcgen05 / TMA kernels, csrc/cuda/gru_persistent.h). These
 * need no initialised group. All tensors fp32 on the current device; `workspace` =
 * bc_gru_workspace_bytes() bytes of scratch, `sync` = 256 zeroed uint32, `status` = 1 uint32 that
 * receives a non-zero code if a bounded wait ran out. `stream` is a cudaStream_t. */
long long bc_gru_workspace_bytes(int T, int B, int H, int ndir);
int bc_gru_supported(int device, int T, int B, int H, int ndir);
/* Tuning aid: device buffer of 8 x T uint64 that block (0,0) of later launches fills with time stamps; NULL = off. */
int bc_gru_set_profile(void* stamps);
int bc_gru_forward(int T, int B, int H, int ndir, const float* w_hh, const float* b_hh, const float* gx, float* y, float* rsv,
                   float* workspace, unsigned* sync, unsigned* status, double timeout_s, void* stream);
int bc_gru_backward(int T, int B, int H, int ndir, const float* w_hh_t, const float* y, const float* rsv, const float* dy,
                    float* dgx, float* dgh, float* workspace, unsigned* sync, unsigned* status, double timeout_s, void* stream);

/* Training-mode batch normalisation of [N, C, HW] fp32 activations fused with the clipped ReLU behind it
 * (y = clamp(bn(x), 0, clip_hi)); csrc/cuda/bn_clip.h. `acc` = scratch of 2 * C doubles; running_* may be NULL.
 * These need no initialised group. */
int bc_bn_clip_forward(const float* x, float* y, const float* gamma, const float* beta, float* running_mean, float* running_var,
                       float* save_mean, float* save_rstd, double* acc, int N, int C, int HW, float eps, float momentum, float clip_hi,
                       void* stream);
int bc_bn_clip_backward(const float* x, const float* dy, const float* gamma, const float* beta, const float* save_mean,
                        const float* save_rstd, float* dx, float* dgamma, float* dbeta, double* acc, int N, int C, int HW,
                        float clip_hi, void* stream);

/* Coordinator validation run on synthetic requests (unit tests). Returns the response type. */
int bc_test_validate(int nranks, const int* ops, const int* dtypes, const int* devices, const int* ndims,
                     const long long* shapes, char* err_out, int err_cap, long long* dim0_out);

#ifdef __cplusplus
}
#endif
#endif /* BCOLL_H_ */
