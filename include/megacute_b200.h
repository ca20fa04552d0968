/* C ABI of the B200 persistent-megakernel runtime (libmegacute_b200.so).
 *
 * The reference runtime reaches its device code through one JIT-compiled callable,
 *     compiled(views, insts, waits, arrives, counters, trace, epoch)
 * built in megacute/runtime.py:312-317 and invoked once per step in megacute/runtime.py:383-384
 * (device entry megacute/kernel.py:242-249).  This header is the ahead-of-time replacement of
 * that boundary: plain pointers and sizes, no torch types.  A host runtime (the Python package in
 * this repository, or any other binding) builds the tables and calls these functions.
 *
 * All device pointers are raw CUDA device addresses owned by the caller.  The library allocates
 * only its own tables (instruction words, wait/arrive tables, dependency counters, op
 * descriptors, status, trace); it never allocates or frees caller tensors.
 * Every function returns 0 on success or a negative MK_E_* code; mk_strerror() names it.
 */
#ifndef MEGACUTE_B200_H
#define MEGACUTE_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- device op kinds (one descriptor per graph op; instructions index descriptors) ---------- */
enum {
    MK_OP_GEMV = 1,        /* linear with <= 8 activation rows: weight rows streamed through smem */
    MK_OP_GEMM = 2,        /* tiled linear, optional split-K partial (reduce-add)                   */
    MK_OP_FINALIZE = 3,    /* out = act(ws + bias) + residual; ws = 0                               */
    MK_OP_ELTWISE = 4,     /* unary / binary / swiglu / modulate / rope tiles                       */
    MK_OP_NORM = 5,        /* RMSNorm / LayerNorm rows                                              */
    MK_OP_ATTENTION = 6,   /* prefill flash attention tile                                          */
    MK_OP_ROPE_APPEND = 7, /* decode: rotate q,k of the new token, append k,v                       */
    MK_OP_DECODE_ATTN = 8, /* decode attention over the cache (optionally fused rope+append, split) */
    MK_OP_INCREMENT = 9,   /* pos += 1                                                              */
    MK_OP_GATHER = 10,     /* out[r] = table[ids[r]]: the embedding lookup of a decode step         */
    MK_OP_ARGMAX = 11      /* ids[r] = argmax(x[r]): greedy sampling, column chunks merged in-op    */
};

#define MK_MAX_PTRS 12
#define MK_INST_WORDS 16

/* One graph op as the kernel sees it.  `ptr[k]` is the device byte address of the first element
 * of operand k's view (0 when absent), `ld[k]` its row stride in elements.  The meaning of
 * ptr/i/f per kind is listed in megacute_b200/encode.py next to the code that fills them and in
 * csrc/megakernel.cu next to the code that reads them.  sizeof == 256.
 * For MK_OP_GEMM, ptr[10] and ptr[11] belong to the library: mk_program_set_ops overwrites them
 * (packed weight tiles, tensor maps) when it binds the op to its tcgen05 body; callers that hand
 * descriptors straight to the kernel (mk_launch_noalloc) leave them 0. */
typedef struct mk_op_desc {
    int32_t  kind;
    int32_t  flags;
    int32_t  i[22];
    float    f[4];
    uint64_t ptr[MK_MAX_PTRS];
    int32_t  ld[MK_MAX_PTRS];
} mk_op_desc;

typedef struct mk_caps {
    int32_t sm_count;
    int32_t cc_major, cc_minor;
    int32_t max_smem_optin;     /* bytes of dynamic shared memory one CTA may request */
    int32_t kernel_smem;        /* bytes the megakernel requests                        */
    int32_t kernel_threads;
    int32_t kernel_regs;        /* registers per thread of the non-tracing kernel       */
    int32_t reserved;
} mk_caps;

/* status words written by the device and returned by mk_program_status() */
enum { MK_ST_CODE = 0, MK_ST_CTA, MK_ST_WARP, MK_ST_SEQ, MK_ST_WHERE, MK_ST_A, MK_ST_B, MK_ST_C, MK_ST_WORDS = 16 };
/* MK_ST_CODE values (MK_DEV_BAD_INST: an instruction names no op, or an op kind the kernel does not know;
 * MK_DEV_CHECK: a library built with -DMK_CHECK found a shared-memory barrier in a state its protocol rules out --
 * armed or released twice in one phase -- recorded which (MK_ST_A: barrier, MK_ST_B: parity) and ended the launch
 * instead of going on) */
enum { MK_DEV_OK = 0, MK_DEV_TIMEOUT_COUNTER = 1, MK_DEV_TIMEOUT_BARRIER = 2, MK_DEV_BAD_INST = 3, MK_DEV_CHECK = 4 };

enum {
    MK_OK = 0,
    MK_E_CUDA = -1,          /* a CUDA runtime call failed: see mk_last_cuda_error()        */
    MK_E_ARG = -2,           /* null / out-of-range argument: mk_last_cuda_error() may say which */
    MK_E_ARCH = -3,          /* the device is not compute capability 10.x                    */
    MK_E_DEVICE = -4,        /* the kernel reported an error in the status buffer            */
    MK_E_NOMEM = -5,
    MK_E_TOO_LARGE = -6      /* mk_launch_noalloc: more counters than the static scratch holds */
};

typedef struct mk_program mk_program;

const char* mk_strerror(int code);
/* Detail of the calling thread's latest MK_E_CUDA or MK_E_ARG ("" when there is none). */
const char* mk_last_cuda_error(void);

/* Replaces: torch.cuda.get_device_properties(0).multi_processor_count (runtime.py:234). */
int mk_query(int device, mk_caps* caps);

/* Upload the tables of one compiled graph.  Replaces the table upload and counter / trace
 * allocation of Program.compile (runtime.py:297-305).
 *   insts    [n_insts][16] int32   word 0 = 1 + op index (0 never appears), 1..7 args, 8 = #waits,
 *                                  9 = first wait pair, 10 = #arrives, 11 = first arrive, 12 = seq
 *   waits    [n_waits][2]  int32   (counter, arrivals per launch)
 *   arrives  [n_arrives]   int32   counter ids
 *   grid                            CTAs to launch (normally the SM count, never more: every CTA must be
 *                                  resident at once, a larger grid is MK_E_ARG); CTA c runs
 *                                  instructions c, c + grid, ...
 *   trace_cap                      per-(CTA, role) trace records, 0 = tracing off                 */
int mk_program_create(int device, const int32_t* insts, int n_insts, const int32_t* waits, int n_waits,
                      const int32_t* arrives, int n_arrives, int n_counters, int n_ops, int grid,
                      int trace_cap, mk_program** out);

/* (Re)bind operand addresses: copy n_ops descriptors to the device on `stream`.  Replaces the
 * per-call strided-view tuple of Program._view_tensors (runtime.py:356-369).  Asynchronous (two
 * pinned staging copies are used in turn; the stream is not synchronised).  Before anything is
 * copied every instruction's arguments are checked against the extents its descriptor states
 * (tile, head and split indices, output ranges): MK_E_ARG, with the instruction named by
 * mk_last_cuda_error(), instead of an out-of-bounds access on the device.
 * Every function of a program makes the program's device current for the duration of the call and
 * puts the caller's current device back before it returns. */
int mk_program_set_ops(mk_program* p, const mk_op_desc* ops, int n_ops, void* stream);

/* One launch of the persistent kernel on `stream` (asynchronous).  Replaces
 * self._compiled(views, insts, waits, arrives, counters, trace, epoch) (runtime.py:383-384);
 * the launch epoch is kept inside the program and the counters are cleared only before it would
 * overflow (runtime.py:377-380). */
int mk_launch(mk_program* p, void* stream);

/* Longest time any device-side wait may spin before the launch gives up with MK_DEV_TIMEOUT_*. */
int mk_program_set_timeout(mk_program* p, uint64_t nanoseconds);

/* Synchronise `stream`, copy the 16 status words out, return MK_E_DEVICE if the kernel reported
 * an error (the status is cleared so the program can be reused after mk_program_reset). */
int mk_program_status(mk_program* p, void* stream, int32_t status[MK_ST_WORDS]);

/* Zero the dependency counters and the epoch (after an error, or to resume from saved state). */
int mk_program_reset(mk_program* p, void* stream);

/* Debug / test access to runtime-owned tables (synchronise the stream first). */
int mk_program_epoch(mk_program* p);
/* How many tile-GEMM ops of the last mk_program_set_ops() run on the tcgen05 tensor cores with
 * bulk-tensor-copied operands (the others, if any, run the mma.sync body: K range per instruction
 * not a multiple of 64, unaligned operands, or MEGACUTE_B200_NO_TCGEN05 set). */
int mk_program_tcgen05_ops(mk_program* p);
/* ... and how many prefill attention ops (head_dim 64; the others run the mma.sync body). */
int mk_program_tcgen05_attention_ops(mk_program* p);
/* Device memory the program holds for tile-image copies of the weights of those ops (made by
 * mk_program_set_ops unless MEGACUTE_B200_NO_WEIGHT_PACK is set, when a weight matrix is bound
 * for the first time; kept while that matrix stays bound; a copy that is no longer bound is not
 * counted here and is freed once every launch enqueued before the rebind has finished).  The copies
 * are snapshots of the weights. */
long long mk_program_packed_bytes(mk_program* p);
/* After changing weights in place: drop the packed copies (synchronises `stream`); the next
 * mk_program_set_ops packs again. */
int mk_program_refresh_weights(mk_program* p, void* stream);
int mk_program_read_counters(mk_program* p, int32_t* out, int n);
int mk_program_read_trace(mk_program* p, int64_t* out, size_t n_words);
int mk_program_clear_trace(mk_program* p, void* stream);
/* Overwrite one (counter, target) wait pair: host-side fault injection for the timeout tests. */
int mk_program_poke_wait(mk_program* p, int wait_index, int counter, int target);

void mk_program_destroy(mk_program* p);

/* One launch that allocates nothing.  (No counterpart in the reference, whose runtime always
 * allocates its counters through torch.)
 *
 * For hosts that cannot call cudaMalloc: a server whose own pool already owns all device memory,
 * or a loop that cannot take the device-wide synchronisation an allocation implies.  The
 * dependency counters and status words -- the only memory the kernel needs beyond the caller's
 * tensors and tables -- live in a static device array inside the library instead
 * (MK_NOALLOC_MAX_COUNTERS counters; about 64 KB held by every GPU that loads the library until
 * the process exits).  A graph that needs more counters is refused with MK_E_TOO_LARGE.
 *
 *   d_insts / d_waits / d_arrives / d_ops   the same tables as mk_program_create / mk_program_set_ops,
 *                                           but already in DEVICE memory owned by the caller
 *   status                                  NULL: return right after the launch is enqueued;
 *                                           else: wait for `stream`, copy the 16 status words here
 *                                           and return MK_E_DEVICE if the kernel reported an error
 *
 * Calls no cudaMalloc / cudaFree or other allocating routine.  The first call on a device looks up
 * the array's address and sets the kernel's shared-memory attribute, so make that first call
 * outside any stream capture.  Every call on a device shares the one array and starts by clearing
 * the counters it uses on `stream`; two calls whose kernels may overlap on the GPU (different
 * streams) race on it -- serialise them.  Split-KV workspaces named by the descriptors must be zero
 * on entry, as for mk_launch.  The wait and arrival tables are device memory the library cannot read:
 * every counter id in them must be below n_counters (mk_program_create checks this for its host
 * tables; here it is the caller's precondition).  grid must not exceed the device's SM count.  The
 * caller's current device is unchanged on return. */
#define MK_NOALLOC_MAX_COUNTERS 16384
int mk_launch_noalloc(int device, const int32_t* d_insts, int n_insts, const int32_t* d_waits, int n_waits,
                      const int32_t* d_arrives, int n_arrives, const mk_op_desc* d_ops, int n_ops,
                      int n_counters, int grid, void* stream, int32_t status[MK_ST_WORDS]);

/* Status words of the latest mk_launch_noalloc on `device`, for callers that passed status == NULL
 * there: waits for `stream`, copies the 16 words out, MK_E_DEVICE if the kernel reported an error.
 * Allocates nothing.  (No counterpart in the reference.) */
int mk_noalloc_status(int device, void* stream, int32_t status[MK_ST_WORDS]);

/* Greedy sampling: out[r] = index of the largest element of row r of `logits` (rows x cols, leading
 * dimension ld in elements; dtype 0 bf16 with ld % 8 == 0 and a 16-byte aligned base, 1 fp32), ties to
 * the lowest index, NaN never selected.  Asynchronous on `stream`; `out` is device memory of `rows`
 * int64.  Replaces the torch argmax of the reference's decode loop (examples/llama/llama1b.py:105),
 * which reduces a 128 256-wide row in a single 512-thread block.  Allocates nothing (its scratch is a
 * static device array); two calls whose kernels may overlap on the GPU share it: serialise them. */
int mk_argmax(const void* logits, int dtype, int rows, int cols, long long ld, long long* out, void* stream);

#ifdef __cplusplus
}
#endif
#endif
