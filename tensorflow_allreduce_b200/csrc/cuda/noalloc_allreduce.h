/* Allreduce over a group of buffers on one GPU for callers that must not allocate.
 *
 * This entry point has no counterpart in the reference: it is an addition of this library.
 *
 * Who needs it: code that runs where device memory cannot be requested any more. Typical cases
 * are a serving engine that handed the whole GPU to its own pool at start-up (a later cudaMalloc
 * simply fails or fragments the pool's budget), and latency-critical loops in which the implicit
 * device-wide synchronisation of cudaMalloc / cudaFree would stall every stream. The other
 * group-on-one-GPU entry points (bc_emu_create / bc_emu_allreduce) allocate their buffers, signal
 * pads and counters with cudaMalloc; this one needs nothing but what the caller passes in.
 *
 * What it does: out[r][i] = scale * sum over q of in[q][i], for r, q in [0, nranks), i in
 * [0, count): the same two-phase kernel as bc_emu_allreduce, launched once, cooperatively, on
 * `stream`. The inputs are left untouched. `scale` applies to the floating-point element types
 * only; for int32, int64 and uint8 the result is the plain sum and `scale` is ignored.
 *
 * Where the scratch lives: in a fixed array inside the library's device image
 * (BC_STATIC_SCRATCH_BYTES = 8,536,320 bytes, about 8.1 MiB). Every GPU on which the library's code gets loaded
 * carries that array until the process exits. It holds, per rank, a 1 MiB staging copy of the
 * input plus the barrier flags and counters of the kernel. Therefore:
 *   - nranks <= 8 and count * sizeof(element) <= BC_STATIC_MAX_BYTES_PER_RANK (1 MiB); larger
 *     requests are refused with an error, nothing is launched (the check is made on `count`
 *     before any multiplication, so a huge count cannot wrap around into a small byte size);
 *   - all calls on a device share the one array. It keeps whatever the previous call left there,
 *     so each call first clears the flags and counters on `stream`; two calls that may overlap
 *     on the GPU (different streams without an ordering between them, or several host threads)
 *     would use the same flags and staging area at once and corrupt each other. Serialise them.
 *
 * First call on a device: the entry point looks up the device address of the array
 * (cudaGetSymbolAddress) and remembers it for that device. Make this first call outside any
 * stream capture, e.g. once during start-up.
 *
 * Pointers: `ins` and `outs` are host arrays of `nranks` device pointers, each 16-byte aligned,
 * all on the current device. The byte range of an output may overlap neither the range of any
 * input nor the range of another output; such a call is refused. `status_out` is device memory
 * for one 32-bit word and is required (NULL is refused): it is set to zero first and receives a
 * non-zero code if a wait inside the kernel ran into its time limit. The kernel then returns
 * without finishing and the outputs are incomplete, so a caller that cannot read this word has no
 * way to tell a good result from a bad one; that is why the word is not optional.
 * `blocks` is the number of thread blocks per rank (0 picks a default); it is limited by what the
 * device can keep resident at once for nranks * blocks blocks of 512 threads.
 *
 * dtype codes as everywhere in this library: 0 float32, 1 int32, 2 int64, 3 bfloat16, 4 float16,
 * 5 float64, 6 uint8. Returns 0 on success, -1 on refusal or launch failure; the reason is then
 * written, NUL-terminated, into `err` (a caller-owned buffer of `err_cap` bytes; may be NULL).
 *
 * The function itself calls neither cudaMalloc nor cudaFree nor any routine that allocates
 * device or pinned memory.
 */
#ifndef BCOLL_NOALLOC_ALLREDUCE_H_
#define BCOLL_NOALLOC_ALLREDUCE_H_

#define BC_STATIC_MAX_RANKS 8
#define BC_STATIC_MAX_BYTES_PER_RANK (1 << 20)
/* Size of the static device array: per rank one staging area, 512 x 8 barrier flags and 512
 * barrier counters of 4 bytes each, plus 256 bytes that hold a spare status word. The .cu file
 * checks this figure against the layout that it really uses. */
#define BC_STATIC_SCRATCH_BYTES \
  (BC_STATIC_MAX_RANKS * (BC_STATIC_MAX_BYTES_PER_RANK + 512 * 8 * 4 + 512 * 4) + 256)

#ifdef __cplusplus
extern "C" {
#endif

int bc_group_allreduce_static(int nranks, const void* const* ins, void* const* outs, long long count, int dtype,
                              float scale, int blocks, unsigned* status_out, void* stream, char* err, int err_cap);

#ifdef __cplusplus
}
#endif
#endif /* BCOLL_NOALLOC_ALLREDUCE_H_ */
