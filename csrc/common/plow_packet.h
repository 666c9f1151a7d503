/* Packet ABI: the on-disk container and the fixed-stride device ISA shared by the compiler
 * (Python writer), the CPU interpreter (C++) and the sm_100a executor.
 *
 * A packet holds a tensor table, named metadata sections and one *program* per row count
 * (prefill buckets and decode rungs).  A program is
 *     insts[]    64-byte fixed-stride instructions in topological order,
 *     stream[]   24-byte entries: which slice range of which instruction a compute unit runs,
 *                concatenated per compute unit (cu_ofs[] indexes it),
 *     waits[]    (counter, target) pairs an entry polls before it may run,
 *     succs[]    counters an entry bumps after its slices are globally visible.
 * Execution model of every backend: spin on wait counters -> run slices -> fence -> bump
 * successor counters.
 *
 * The same role is played in the reference by runtime/common/dev_isa.h:1579-1613,1698-1707
 * (PlowWait / PlowDevInst / PlowStreamEnt) and dev_blob.h:14-28 (PLOWDEV container); field
 * sizes are kept (64-byte instruction with 3 scalar words, 8 u16 tensor handles and 8 u32
 * immediates), the opcode space and container layout are this project's own.
 */
#ifndef PLOW_PACKET_H
#define PLOW_PACKET_H
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define PLOW_PKT_MAGIC "PLOWB200"
#define PLOW_PKT_VERSION 3u
#define PLOW_CTR_STRIDE_U32 32u /* one counter per 128-byte line */
#define PLOW_KV_PAGE 64u
#define PLOW_T_NONE 0xFFFFu
#define PLOW_EXPERT_UNUSED 0xFFFFFFFFu

/* ---- opcodes ------------------------------------------------------------------------- */
typedef enum PlowOp {
  PLOW_OP_NOP = 0,
  /* dense core */
  PLOW_OP_EMBED = 1,          /* t0=out[rows,H] t1=table t2=in.ids ; f0=scale */
  PLOW_OP_RMSNORM = 2,        /* t0=out t1=x t2=gamma(opt) ; f0=eps i0=H i1=gamma_mode(0 g,1 1+g) */
  PLOW_OP_ADD_NORM = 3,       /* t0=out t1=resid(in/out) t2=delta t3=gamma ; resid+=delta; out=norm(resid) */
  PLOW_OP_GEMM = 4,           /* t0=y t1=x t2=w t3=resid(opt) t4=sx t5=sw t7=bias(opt) ; i0=N i1=K i2=flags */
  PLOW_OP_ROPE_KV = 5,        /* t0=q out t1=fused qkv rows t2=kcache t3=vcache t4=qnorm(opt) t5=knorm(opt) t6=rope table
                                 t7=gate out (i7=1: query heads are [Q | gate] pairs) or the e4m3 cache's scales [P,64,2*nkv]
                                 i0=nq i1=nkv i2=hd i3=rot_dim i4=pair_mode i5=layer i6=gamma_mode i7=gated ; f0=eps */
  PLOW_OP_ATTN = 6,           /* t0=out t1=q t2=kcache t3=vcache t4=e4m3 cache scales (opt) t5=sinks [nq] f32 (opt: one extra
                                 logit per head in every softmax, no value) ;
                                 i0=nq i1=nkv i2=hd i3=window i4=mode i5=layer; f0=scale */
  PLOW_OP_ROW_GATHER = 7,     /* t0=out[nsample,H] t1=x t2=in.sample_rows */
  PLOW_OP_ARGMAX = 8,         /* t0=out.ids t1=logits ; i0=V */
  PLOW_OP_SAMPLE = 9,         /* t0=out.ids t1=logits t2=in.sampling ; i0=V */
  PLOW_OP_RESIDUAL = 10,      /* t0=out t1=a t2=b */
  PLOW_OP_GLU = 11,           /* t0=out t1=gate t2=up ; i0=activation (0 silu, PLOW_GEMM_ACT_GELU_*) : out = act(gate) * up */
  PLOW_OP_QUANT_ACT = 12,     /* t0=q t1=scales t2=x ; i0=K */
  /* MLA */
  PLOW_OP_MLA_KV_WRITE = 20,  /* latent norm + k_rope rope + cache write */
  PLOW_OP_MLA_Q_ROPE = 21,
  PLOW_OP_MLA_DECODE = 22,    /* absorbed decode over the latent cache */
  PLOW_OP_MLA_PREFILL = 23,   /* materialised K/V flash prefill */
  PLOW_OP_MLA_ABSORB_Q = 24,  /* q_nope * W_uk -> latent-space query */
  PLOW_OP_MLA_FOLD_V = 25,    /* o_latent * W_uv -> per-head v */
  /* DSA */
  PLOW_OP_DSA_INDEX = 30,     /* indexer scores */
  PLOW_OP_DSA_TOPK = 31,      /* exact top-k select */
  /* MoE */
  PLOW_OP_ROUTER_TOPK = 40,   /* t0=table{eid,gate} t1=logits t2=bias ; i0=E i1=k i2=n_group i3=topk_group i4=flags ; f0=route_scale */
  PLOW_OP_MOE_ALIGN = 41,     /* histogram/sort rows by expert */
  PLOW_OP_MOE_GATHER = 42,    /* gather (and quantise) rows into expert order */
  PLOW_OP_MOE_GEMM = 43,      /* grouped GEMM */
  PLOW_OP_MOE_COMBINE = 44,   /* out = resid + shared + sum_j gate_j * part_j (fixed slot order) */
  /* gated delta rule */
  PLOW_OP_GDN_CONV = 50,
  PLOW_OP_GDN_GATES = 51,
  PLOW_OP_GDN_STEP = 52,
  PLOW_OP_GDN_CHUNK = 53,
  PLOW_OP_GATED_NORM = 54,
  PLOW_OP_SIGMOID_GATE = 55,
  /* collectives */
  PLOW_OP_XREDUCE = 60,          /* all-reduce over peer memory */
  PLOW_OP_XREDUCE_ADD_NORM = 61, /* all-reduce + residual + RMSNorm */
  PLOW_OP_XGATHER = 62,          /* all-gather */
  PLOW_OP_XREDUCE_SCATTER = 63,
  PLOW_OP_XA2A_DISPATCH = 64,    /* expert-parallel token dispatch */
  PLOW_OP_XA2A_COMBINE = 65,     /* expert-parallel combine */
  PLOW_OP_XARGMAX_FIN = 66,      /* vocab-sharded argmax fold */
  PLOW_OP_GEMM_XREDUCE = 67,     /* fused GEMM -> all-reduce */
  PLOW_OP_XGATHER_GEMM = 68,     /* fused all-gather -> GEMM */
  PLOW_OP__COUNT = 69
} PlowOp;

/* GEMM flags (i2) */
#define PLOW_GEMM_DUAL_SILU 1u   /* w = [gate; up]; y = silu(x gate^T) * (x up^T) */
#define PLOW_GEMM_FP8_BLOCK 2u   /* e4m3 operands, 1x128 / 128x128 fp32 scales */
#define PLOW_GEMM_OUT_F32 4u
#define PLOW_GEMM_RESIDUAL 8u
#define PLOW_GEMM_QUANT_OUT 16u
#define PLOW_GEMM_ACT_GELU_TANH 32u /* with DUAL: gelu (tanh form) instead of silu on the gate */
#define PLOW_GEMM_ACT_GELU_ERF 64u  /* with DUAL: gelu (erf form) */
#define PLOW_GEMM_BIAS 128u         /* t7 = bias [N] (f32 in f32 packets, else bf16), added to the fp32 sum before the store */

/* attention modes (i4) */
#define PLOW_ATTN_CAUSAL 0u      /* token-batch rows, each attends to its sequence up to pos */
#define PLOW_ATTN_DECODE 1u      /* one row per sequence */

/* dtypes */
typedef enum PlowDType { PLOW_F32 = 0, PLOW_BF16 = 1, PLOW_F16 = 2, PLOW_E4M3 = 3, PLOW_I32 = 4, PLOW_U8 = 5, PLOW_I64 = 6 } PlowDType;

/* tensor classes: who provides the storage */
typedef enum PlowTClass {
  PLOW_TC_WEIGHT = 0,   /* bound from the checkpoint by name */
  PLOW_TC_DERIVED = 1,  /* computed at load from checkpoint tensors (cat/, fp8/ twins, absorbed MLA) */
  PLOW_TC_GEN = 2,      /* generated at load (RoPE tables) */
  PLOW_TC_KV = 3,       /* paged KV pool */
  PLOW_TC_STATE = 4,    /* recurrent state slots */
  PLOW_TC_ACT = 5,      /* activation arena (offset assigned by the planner) */
  PLOW_TC_INPUT = 6,    /* per-step host inputs (ids, pos, page table ...) */
  PLOW_TC_OUTPUT = 7,   /* per-step results read by the host */
  PLOW_TC_PEER = 8      /* symmetric peer-visible buffer */
} PlowTClass;

/* ---- instruction stream -------------------------------------------------------------- */
typedef union PlowWord { float f; uint32_t u; int32_t i; } PlowWord;

typedef struct PlowInst {
  uint16_t op;      /* PlowOp */
  uint16_t nslice;  /* number of independent slices the op is cut into */
  PlowWord w[3];    /* f0..f2 */
  uint16_t t[8];    /* tensor handles, PLOW_T_NONE when absent */
  uint32_t i[8];    /* integer immediates */
} PlowInst;         /* 64 bytes */

typedef struct PlowStreamEnt {
  uint32_t inst;      /* instruction index */
  uint16_t slice0;    /* first slice */
  uint16_t nslice;    /* slices run by this entry */
  uint32_t wait_ofs;  /* into waits[] */
  uint32_t succ_ofs;  /* into succs[] */
  uint16_t n_wait;
  uint16_t n_succ;
  uint32_t seg;       /* segment id (launch unit) */
} PlowStreamEnt;      /* 24 bytes */

typedef struct PlowWait { uint32_t ctr; uint32_t target; } PlowWait; /* 8 bytes */

/* device trace record, one per stream entry (slot = stream index, no atomics) */
typedef struct PlowTraceRec {
  uint32_t cu, pc, inst, op;
  uint64_t t_arrive, t_ready, t_end;
} PlowTraceRec; /* 40 bytes */

/* ---- container ----------------------------------------------------------------------- */
typedef struct PlowPktHeader {
  char magic[8];
  uint32_t version;
  uint32_t header_bytes;
  uint32_t n_tensor;
  uint32_t n_program;
  uint32_t n_section;
  uint32_t n_cu;            /* compute units the streams were planned for */
  uint64_t tensor_ofs;      /* PlowTensorEnt[n_tensor] */
  uint64_t program_ofs;     /* PlowProgramEnt[n_program] */
  uint64_t section_ofs;     /* PlowSectionEnt[n_section] */
  uint64_t strtab_ofs;
  uint64_t strtab_bytes;
  uint64_t file_bytes;
  uint64_t act_arena_bytes; /* max over programs */
  uint8_t content_hash[32]; /* sha256 of everything after the header */
} PlowPktHeader;            /* 120 bytes */

typedef struct PlowTensorEnt {
  uint32_t name_ofs;   /* into strtab */
  uint16_t dtype;      /* PlowDType */
  uint16_t tclass;     /* PlowTClass */
  uint16_t rank;
  uint16_t flags;
  uint32_t shard_axis; /* 0xFFFFFFFF replicated */
  int64_t dims[4];     /* -1 = rows of the running program */
  uint64_t arena_ofs;  /* ACT tensors: offset in the activation arena (per program table overrides) */
  uint64_t bytes;      /* fixed-size tensors; 0 when row dependent */
} PlowTensorEnt;       /* 64 bytes */

typedef enum PlowProgRole { PLOW_ROLE_PREFILL = 0, PLOW_ROLE_DECODE = 1, PLOW_ROLE_MIXED = 2 } PlowProgRole;

typedef struct PlowProgramEnt {
  uint32_t role;       /* PlowProgRole */
  uint32_t rows;       /* row count the program was planned for */
  uint32_t rank;       /* tensor/expert-parallel rank */
  uint32_t n_inst;
  uint32_t n_stream;
  uint32_t n_wait;
  uint32_t n_succ;
  uint32_t n_ctr;
  uint32_t n_cu;
  uint32_t n_seg;
  uint64_t inst_ofs;
  uint64_t stream_ofs;
  uint64_t cu_ofs;     /* uint32[n_cu+1] */
  uint64_t wait_ofs;
  uint64_t succ_ofs;   /* uint32[n_succ] counter ids */
  uint64_t actmap_ofs; /* uint64[n_tensor] arena offsets for this program (UINT64_MAX unused) */
  uint64_t arena_bytes;
} PlowProgramEnt;      /* 96 bytes */

typedef struct PlowSectionEnt {
  uint32_t name_ofs;
  uint32_t kind;       /* 4 = named metadata (JSON) */
  uint64_t ofs;
  uint64_t bytes;
} PlowSectionEnt;      /* 24 bytes */

#ifdef __cplusplus
}
static_assert(sizeof(PlowInst) == 64, "PlowInst must be 64 bytes");
static_assert(sizeof(PlowStreamEnt) == 24, "PlowStreamEnt must be 24 bytes");
static_assert(sizeof(PlowWait) == 8, "PlowWait must be 8 bytes");
static_assert(sizeof(PlowTraceRec) == 40, "PlowTraceRec must be 40 bytes");
static_assert(sizeof(PlowPktHeader) == 120, "PlowPktHeader must be 120 bytes");
static_assert(sizeof(PlowTensorEnt) == 64, "PlowTensorEnt must be 64 bytes");
static_assert(sizeof(PlowProgramEnt) == 96, "PlowProgramEnt must be 96 bytes");
static_assert(sizeof(PlowSectionEnt) == 24, "PlowSectionEnt must be 24 bytes");
#endif
#endif /* PLOW_PACKET_H */
