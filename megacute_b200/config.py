"""Constants shared by the host scheduler and the CUDA kernel (mirrored in csrc/mk_device.cuh and include/megacute_b200.h).

The reference keeps its equivalents in ``megacute/config.py`` (CTA shape, tile sizes, instruction
word layout) and ``megacute/runtime.py:28-29`` (split cost model); the values here are this
runtime's own choices.
"""

# ---- CTA shape: 8 compute warps + 1 producer warp that streams weights ahead of them + 1 finisher warp
COMPUTE_WARPS = 8
COMPUTE_THREADS = 32 * COMPUTE_WARPS
NUM_THREADS = COMPUTE_THREADS + 96     # + producer warp + finisher warp + feeder warp

# ---- weight-streaming GEMV path (linear with <= 8 activation rows)
GEMV_MAX_ROWS = 8
GEMV_XBUF_BYTES = 65536         # fp32 copy of the activation rows held in shared memory
GEMV_ROWS_PER_STAGE = 16        # weight rows per ring stage
GEMV_SEGMENT = 2048             # elements of a weight row per stage (one 4 KB bulk copy)
GEMV_STAGE_BYTES = GEMV_ROWS_PER_STAGE * (GEMV_SEGMENT * 2 + 16)
GEMV_STAGES = 2

# ---- tile GEMM path
GEMM_BM, GEMM_BN, GEMM_BK = 128, 128, 32
MIN_SPLIT_KTILES = 8            # k-tiles (of GEMM_BK) per K split
MAX_K_SPLITS = 8
INST_US, SM_GBPS = 2.0, 40.0    # split-K cost model: fixed us per instruction, GB/s one SM draws from HBM
# 256-wide output tiles (one activation k-tile feeds two weight tiles) for ops with more than WIDE_MIN_ROWS rows:
# us per 64-element k-tile of a 128 x 128 / 128 x 256 tile and us per epilogue, from the kernel's timeline (two issuing
# threads; a 128 x 256 k-tile is one 32 KB weight slot and one N = 256 instruction per 16 K-elements)
GEMM_BN_WIDE, WIDE_MIN_ROWS = 256, 128
KTILE_US, KTILE_US_WIDE, EPILOGUE_US, EPILOGUE_US_WIDE = 0.27, 0.42, 3.5, 7.0

# ---- pointwise / norm / attention tiling
EW_ROWS, EW_COLS = 32, 512
FINALIZE_MIN_ROWS, FINALIZE_MIN_INSTS = 4, 96     # SplitFinalize: shorter tiles until the op has this many instructions
NORM_ROWS = COMPUTE_WARPS       # rows per norm instruction (one per warp); 1 when the op has few rows
WIDE_NORM_ROWS = 256
ROPE_APPEND_ROWS = COMPUTE_WARPS
ATTN_BQ, ATTN_BK = 128, 64
DECODE_KEYS_PER_TILE = 64
MIN_SPLIT_KEYS = 64
MAX_KV_SPLITS = 32
DECODE_MERGE_BYTES = 88 * 1024   # shared memory the merging split may fill with partial rows
# split-KV cost model (us): per instruction; partials + merge when split (base, per split); per key tile
DEC_FIXED_US, DEC_MERGE_US, DEC_MERGE_US_PER_SPLIT, DEC_TILE_US = 4.0, 1.0, 0.05, 1.1
# of the fixed cost, the part an instruction pays once however many kv heads it handles (fetch, dependency wait, arrival)
DEC_SHARED_US = 2.5
# many-sequence form (one instruction = a sequence's KV split over all kv heads, whole rows through bulk copies),
# constants measured on B200 at batch 64 (contexts 256 .. 32K, 1 .. 30 splits): used from BULK_MIN_BATCH sequences
# on, or from BULK_MIN_BATCH_LONG when the cache is at least BULK_LONG_SEQ rows long (batch 8 and 16 at context
# 1K were 5 - 10 % faster in the per-head form: more instructions to spread, and the stream is short);
# us per 16-row tile per KB of cache row (all SMs streaming: the HBM rate); us per instruction = max(fixed, per split x S - 3)
BULK_MIN_BATCH, BULK_MIN_BATCH_LONG, BULK_LONG_SEQ = 32, 8, 8192
BULK_TILE_US_PER_KB, BULK_FIXED_US, BULK_US_PER_SPLIT = 0.745, 3.0, 0.8
BULK_TILE_ROWS = 16

# ---- instruction word layout (16 x int32)
IW = 16
W_OP = 0                        # 0 = stop, else 1 + op index
W_ARG0 = 1                      # args in words 1..7
N_ARGS = 7
W_NWAIT, W_WAIT_OFF = 8, 9      # wait table slice: pairs (counter, target)
W_NARRIVE, W_ARRIVE_OFF = 10, 11
W_SEQ = 12                      # global instruction index

# ---- device op kinds (include/megacute_b200.h: MK_OP_*)
OP_GEMV, OP_GEMM, OP_FINALIZE, OP_ELTWISE, OP_NORM, OP_ATTENTION, OP_ROPE_APPEND, OP_DECODE_ATTN, OP_INCREMENT, \
    OP_GATHER, OP_ARGMAX = range(1, 12)
GATHER_ROWS = 8                 # rows per gather instruction (one per compute warp)
ARGMAX_MAX_CHUNKS = 256         # column chunks per row of an argmax (the merging instruction takes one partial per thread)

ACT_CODE = {None: 0, "identity": 0, "relu": 1, "silu": 2, "gelu_tanh": 3, "gelu": 3, "exp": 4, "neg": 5,
            "sigmoid": 6, "square": 7, "swiglu": 8}
BINARY_CODE = {"add": 0, "sub": 1, "mul": 2, "max": 3, "min": 4}
EW_UNARY, EW_BINARY, EW_SWIGLU, EW_MODULATE, EW_ROPE, EW_GATED = range(6)
