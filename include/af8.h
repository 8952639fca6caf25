/*
 * af8.h -- C ABI of libaf8: the fused optimizer step over block-quantised
 * states (AL8/AL16 second moments, UF8/UF4/d8/d4 momentum) for NVIDIA B200
 * (sm_100a).
 *
 * The library replaces the reference's pybind11 module `adafactor8bit_cuda`
 * (kernels.cu:3088-3151).  Where the reference passes torch::Tensor objects and
 * launches one kernel per parameter tensor, this ABI takes raw device
 * pointers, 64-bit sizes and a stream, and every step entry point works on a
 * whole TABLE of tensors in one launch.
 *
 * Conventions
 *   - every function returns AF8_OK (0) or an AF8_ERR_* code; af8_last_error()
 *     returns the message of the calling thread's last failure;
 *   - `stream` is a cudaStream_t passed as void*; all work is enqueued on it and
 *     no entry point synchronises the device (except af8_device_status and
 *     af8_device_status_clear, which say so);
 *   - the caller owns all memory.  What the library keeps on a device between calls:
 *     the two dynamic-map codebooks in constant memory, the sticky error flag that
 *     af8_device_status reads, and the fixed 1 MiB array of
 *     af8_fullrank_limited_step_noalloc;
 *   - tensor tables (`af8_*_tensor` arrays) live in DEVICE memory; they are
 *     filled on the host and copied by the caller;
 *   - the current device must be the one that owns the pointers.
 */
#ifndef AF8_H
#define AF8_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define AF8_VERSION 1

#if defined(__GNUC__)
#define AF8_API __attribute__((visibility("default")))
#else
#define AF8_API
#endif

/* return codes */
enum {
    AF8_OK = 0,
    AF8_ERR_INVALID = 1,      /* bad argument (null pointer, size, enum, alignment) */
    AF8_ERR_UNSUPPORTED = 2,  /* valid request that this build has no kernel for */
    AF8_ERR_CUDA = 3          /* a CUDA runtime call or a kernel launch failed */
};

/* element types of parameters and gradients */
enum { AF8_F32 = 0, AF8_BF16 = 1, AF8_F16 = 2 };

/* second-moment / confidence state formats (v_quant_type, c_quant_type;
 * optimizer.py:25) */
enum { AF8_V_FP32 = 0, AF8_V_AL8 = 8, AF8_V_AL16 = 16,
       AF8_V_NONE = 1 };  /* no second moment: the SGD mode (beta2 and beta2_decay both None) */

/* momentum state formats (m_quant_type; optimizer.py:24); NONE = beta1 is None */
enum { AF8_M_NONE = 0, AF8_M_UF8 = 1, AF8_M_UF4 = 2, AF8_M_D8 = 3, AF8_M_D4 = 4, AF8_M_FP32 = 5 };

/* pass selection; mirrors the reference's NOCLIP / NORM / APPLY kernel modes
 * (_dispatch_cuda_clip, optimizer.py:1048-1077) */
enum {
    AF8_MODE_NOCLIP = 0,  /* single pass: update states and parameters */
    AF8_MODE_SUMSQ = 1,   /* first pass: per-block sum of squares of the update, no writes
                             to states or parameters */
    AF8_MODE_APPLY = 2,   /* second pass: as NOCLIP, scaled by af8_dyn_scalars */
    AF8_MODE_SUMSQ_M = 3, /* momentum-only rule, second statistic pass: sum of squares of
                             the new momentum (reads af8_dyn_scalars.pre_div), no writes */
    AF8_MODE_LAG = 4      /* single pass with the previous step's norm (lag_norm=True, optimizer.py:1056-1071;
                             kernels.cu:651-656): updates states and parameters with the af8_dyn_scalars that
                             af8_lag_scalars(phase 0) prepared and writes this step's partial sums of squares
                             of the raw update for af8_lag_scalars(phase 1) */
};

AF8_API int af8_version(void);
AF8_API const char *af8_last_error(void);

/* sizeof() of the i-th structure of this header as the library was compiled, in the order
 * fullrank_tensor, dyn_scalars, fullrank_cfg, norm_tensor, scale_tensor, small_state,
 * factored_tensor, factored_cfg, apollo_scalars_in, apollo_scalars, apollo_proj_desc,
 * apollo_finish_tensor, lag_tensor; -1 for any other index.
 * A binding checks its own mirrors against these when it loads the library. */
AF8_API int32_t af8_struct_size(int32_t index);

/* Device-side health: waits inside the kernels (on asynchronous copies) are
 * bounded; a wait that ran out sets a sticky flag on the device instead of
 * hanging.  This call synchronises `stream` and returns the flag of the current
 * device in *status_out: 0 = healthy, 1 = an asynchronous copy never completed
 * (results of that launch are invalid).  No counterpart in the reference. */
AF8_API int af8_device_status(int32_t *status_out, void *stream);
/* Reset that flag to 0 (synchronises `stream`).  No counterpart in the reference. */
AF8_API int af8_device_status_clear(void *stream);
/* Self-test of the bounded waits: a one-thread kernel arms an mbarrier for more bytes than the single
 * 32-byte copy from `src32` (device memory, 16-byte aligned) delivers and waits for at most limit_ns
 * (1 .. 1e9).  Nothing stays in flight and nothing faults; the wait has to give up, writes 1 to
 * *gave_up_dev (device int32) and raises the device flag with the code of a copy time-out, which
 * af8_device_status then reports until af8_device_status_clear.  No counterpart in the reference. */
AF8_API int af8_selftest_bounded_wait(const void *src32, int64_t limit_ns, int32_t *gave_up_dev, void *stream);

/* Upload the signed dynamic-map codebooks (256 and 16 sorted entries) used by
 * the d8 / d4 momentum formats to the current device.
 * Replaces set_qmap (kernels.cu:32-37, optimizer.py:109-133). */
AF8_API int af8_set_qmap(const float *host_map8, const float *host_map4, void *stream);

/* ------------------------------------------------------------------------ */
/* Full-rank step: AdamW / RMSprop / unfactored Adafactor                    */
/* ------------------------------------------------------------------------ */

/* Per-tensor scalars that a first pass produces on the device and the APPLY
 * pass consumes (written by af8_norm_finalize). */
typedef struct af8_dyn_scalars {
    float step;       /* -alpha / denom: multiplier of the update in p += step*u */
    float fira;       /* Fira scale applied to the update before `step` */
    float pre_div;    /* divisor of u_t before the momentum EMA (momentum-only path) */
    float zero;       /* non-zero: the update norm was not finite, use a zero update */
    float norm;       /* the norm that was measured (diagnostic, read by tests) */
    float reserved[3];
} af8_dyn_scalars;

/* One parameter tensor of a full-rank launch.  The V state is padded to a
 * multiple of `block`, the M state to a multiple of `m_block`, exactly as the
 * reference allocates them (optimizer.py:389-401, 574-590). */
typedef struct af8_fullrank_tensor {
    void *param;            /* numel elements of cfg.param_dtype */
    const void *grad;       /* numel elements of cfg.grad_dtype */
    void *v_q;              /* AL8: uint8, AL16: uint16 codes; NULL for fp32 V */
    float *v_scale;         /* one per V block */
    float *v_min_log;       /* one per V block */
    float *v_f32;           /* fp32 V state (cfg.v_fmt == AF8_V_FP32) */
    uint8_t *m_q;           /* momentum codes (4-bit formats: two per byte) */
    float *m_scale;         /* one per M block */
    float *m_f32;           /* fp32 momentum (cfg.m_fmt == AF8_M_FP32) */
    int64_t numel;
    int64_t first_block;    /* index of this tensor's first V block in the launch */
    /* host scalars of this step, rounded to binary32 as the reference's 0-d
     * tensors are (optimizer.py:2009-2040) */
    float decay;            /* 1 - wd_mult*wd; 1.0 when weight_decay == 0 */
    float alpha;            /* step size with bias correction folded in */
    float v_w;              /* second-moment EMA weight beta_val */
    float v_keep;           /* float(1 - beta_val), used by the fp32 V state (v*v_keep + v_w*g*g, the mul_ / addcmul_
                               form of optimizer.py:2186-2189); a negative value selects Tensor.lerp_(g*g, v_w)
                               instead (APOLLO's fp32 low-rank state, optimizer.py:2797-2799); with AF8_V_NONE:
                               float(1 - beta1), the divisor of the momentum */
    float v_eps_add;        /* float(beta_val * eps_for_grad_sq), fp32 V state */
    float m_w;              /* float(1 - beta1) */
    float eps_gradsq;       /* added to g*g (0 in Adam mode) */
    float eps_denom;        /* added to sqrt(v) in Adam mode */
    float eps_sq;           /* floor of v outside Adam mode */
    float reserved;
    uint64_t sr_base;       /* stochastic rounding: seed * 0x9E3779B97F4A7C15 + step * 0xD1B54A32D192ED03
                               (mod 2^64) with the parameter's state["sr_seed"] and step number
                               (optimizer.py:1889-1892, 2040); element i draws from counter sr_base + i */
    void *param_copy;       /* optional bf16 copy of the updated parameter (numel 16-bit words, 16-byte aligned),
                               written next to the fp32 parameter with round-to-nearest: the compute copy of a
                               mixed-precision run, e.g. this rank's slice of an all-gather buffer.  NULL: none.
                               Only with cfg.param_dtype == AF8_F32.  No counterpart in the reference. */
} af8_fullrank_tensor;

/* Launch-wide configuration: everything that selects a kernel variant. */
typedef struct af8_fullrank_cfg {
    int32_t param_dtype;    /* AF8_F32, AF8_BF16 or AF8_F16.  A 16-bit parameter is rounded to nearest
                               after the weight decay and again after the update, as the reference's
                               in-place ops on such a tensor do, or once, stochastically (below) */
    int32_t grad_dtype;     /* AF8_F32, AF8_BF16 or AF8_F16 */
    int32_t v_fmt;          /* AF8_V_* */
    int32_t m_fmt;          /* AF8_M_* */
    int32_t block;          /* V block size: multiple of 128, >= 128 */
    int32_t m_block;        /* M block size: multiple of 4, >= 32, divides block */
    int32_t use_adam_denom; /* 1: u = m/(sqrt(v)+eps); 0: u = m*rsqrt(max(v,eps_sq)) */
    int32_t momentum_only;  /* 1: momentum is the EMA of the normalised gradient */
    int32_t negate_grad;    /* maximize */
    int32_t mode;           /* AF8_MODE_* */
    float v_floor;          /* lower clamp of a block's min_log (-126 on this path) */
    int32_t stochastic_round; /* 16-bit parameters only: p*decay + step*u is formed in binary32 and rounded
                               stochastically with the counter generator of af8_fullrank_tensor.sr_base
                               (stochastic_round_writeback, optimizer.py:873-881; kernels.cu:48-161) */
} af8_fullrank_cfg;

/* One fused pass over every tensor of the table.
 *   host_tensors  optional host copy of the table (n_tensors entries).  When it
 *                 is not NULL the library validates it (pointer alignment,
 *                 ascending first_block, block count) and enqueues its copy
 *                 into dev_tensors on `stream` before the launch; the host
 *                 memory must stay unchanged until that copy has run.  When it
 *                 is NULL, dev_tensors must already hold a valid table.
 *   dev_tensors   device array of n_tensors entries, first_block ascending
 *   total_blocks  sum over tensors of ceil(numel / cfg.block)
 *   dyn           device array of n_tensors entries; read in the APPLY and
 *                 SUMSQ_M modes, may be NULL in the other modes
 *   block_sumsq   device array of total_blocks floats; written in the SUMSQ
 *                 modes (one partial sum per V block), may be NULL otherwise
 * Pointers of quantised states, parameters and gradients must be 16-byte
 * aligned.
 * Replaces fused_update_1d_{noclip,norm,apply}, fused_update_1d_vonly_* and
 * fused_update_1d_full_* (kernels.cu:826-990, 1100-1255, 1374-1515) and the
 * separate weight-decay pass (optimizer.py:2039). */
AF8_API int af8_fullrank_step(const af8_fullrank_cfg *cfg,
                      const af8_fullrank_tensor *host_tensors,
                      af8_fullrank_tensor *dev_tensors, int32_t n_tensors,
                      int64_t total_blocks, const af8_dyn_scalars *dyn,
                      float *block_sumsq, void *stream);

/* Validate a host table and enqueue its copy into dev_tensors without
 * launching a kernel.  Use it when the device table must be patched (see
 * af8_param_scale) before af8_fullrank_step runs with host_tensors == NULL.
 * No counterpart in the reference, which passes scalars per launch. */
AF8_API int af8_fullrank_upload(const af8_fullrank_cfg *cfg,
                                const af8_fullrank_tensor *host_tensors,
                                af8_fullrank_tensor *dev_tensors, int32_t n_tensors,
                                int64_t total_blocks, void *stream);

/* Per-tensor description for af8_norm_finalize. */
typedef struct af8_norm_tensor {
    int64_t first_block;    /* first entry of block_sumsq that belongs to the tensor */
    int64_t n_blocks;       /* number of entries; or -1: first_block then holds the device ADDRESS of one double,
                               the tensor's whole sum of squares, and block_sumsq is not read for this tensor.
                               That form serves a tensor whose elements are spread over several launch tables or
                               several GPUs: the caller adds up the pieces' partial sums (and all-reduces them)
                               before this call; sqrt_n and clip_div then describe the whole tensor. */
    float *fira_prev;       /* device scalar: previous limited norm (state key
                               "fira_prev_norm"); NULL when the limiter is off */
    int32_t fira_has_prev;  /* 0 on the first limited step of this tensor */
    int32_t pre_div_mode;   /* 0: write step/fira/zero and pre_div = 1
                               1: write pre_div = max((norm/sqrt_n)/d, 1), step = -alpha,
                                  fira = 1 (clip of the momentum-only rule,
                                  optimizer.py:897-899)
                               2: as 0 but leave pre_div untouched */
    float alpha;            /* numerator of `step` */
    float clip_div;         /* float(sqrt(numel)*d); <= 0 disables clipping */
    float sqrt_n;           /* float(sqrt(numel)) */
    float d;
    float fira_margin1;     /* float(1 + fira_margin) */
    int32_t partials_f64;   /* 0: block_sumsq holds floats (full-rank passes); 1: doubles
                               (factored passes) */
    const float *alpha_dev; /* when not NULL: device location of alpha (overrides `alpha`);
                               used when af8_param_scale computed it on the device */
} af8_norm_tensor;

/* Reduce the per-block partial sums of each tensor (fixed order, binary64),
 * take the norm, run the Fira norm-growth limiter and the RMS clip on it and
 * write af8_dyn_scalars for the APPLY pass.  One launch for all tensors.
 * Replaces fira_scalar (kernels.cu:3029-3084) and the host-side tensor
 * arithmetic of _apply_fira_cuda / _safe_rms_denom (optimizer.py:785-793,
 * 859-863). */
AF8_API int af8_norm_finalize(const af8_norm_tensor *tensors, int32_t n_tensors,
                              const void *block_sumsq, af8_dyn_scalars *dyn,
                              void *stream);

/* Per-tensor description for af8_lag_scalars: the one-step-lag variant of clipping and of the
 * limiter (lag_norm=True).  The three device scalars are the reference's state entries
 * "prev_update_norm", "lag_fira_scale" and "fira_prev_norm" (optimizer.py:1056-1071). */
typedef struct af8_lag_tensor {
    int64_t first_block;      /* first entry of block_sumsq that belongs to the tensor */
    int64_t n_blocks;
    float *prev_update_norm;  /* norm of the previous step's raw update; 0 before the first step */
    float *lag_fira_scale;    /* limiter scale computed from the previous step's norm; NULL: limiter off */
    float *fira_prev;         /* "fira_prev_norm"; NULL: limiter off */
    const float *alpha_dev;   /* when not NULL: device location of alpha (overrides `alpha`) */
    float alpha;
    float clip_div;           /* float(sqrt(numel)*d); <= 0 disables clipping */
    float fira_margin1;       /* float(1 + fira_margin) */
    int32_t has_lag_fira;     /* lag_fira_scale holds a value (not the first lagged step) */
    int32_t fira_has_prev;    /* fira_prev holds a value */
    int32_t partials_f64;     /* as af8_norm_tensor.partials_f64 */
    int32_t reserved[2];
} af8_lag_tensor;

/* phase 0, before the AF8_MODE_LAG pass: dyn.step = -(alpha * lag_fira_scale) / denom with
 *          denom = max(1, prev_update_norm / clip_div), fira = 1, zero = 0, pre_div = 1.
 *          (The momentum-only rule is not covered: run its exact passes instead.)
 * phase 1, after it: norm = sqrt(sum of the tensor's partial sums); prev_update_norm = norm;
 *          with the limiter, lag_fira_scale = _compute_fira_scale(norm) and fira_prev is advanced
 *          (optimizer.py:760-782); dyn.norm = norm.
 * Replaces the host-side tensor arithmetic of _dispatch_cuda_clip's lag branch. */
AF8_API int af8_lag_scalars(const af8_lag_tensor *tensors, int32_t n_tensors, int32_t phase,
                            const void *block_sumsq, af8_dyn_scalars *dyn, void *stream);

/* ------------------------------------------------------------------------ */
/* Factored step: Adafactor and CAME on 2-D tensors                          */
/* ------------------------------------------------------------------------ */

/* A small per-row or per-column state: AL8/AL16 codes with per-block ranges,
 * or fp32 (optimizer.py:389-401: keys <prefix>_q/_scale/_min_log or <prefix>). */
typedef struct af8_small_state {
    void *q;            /* uint8 (AL8) / uint16 (AL16) codes, padded to `block`; NULL for fp32 */
    float *scale;
    float *min_log;
    float *f32;         /* fp32 state when fmt == AF8_V_FP32 */
    int32_t fmt;        /* AF8_V_* */
    int32_t block;      /* AL block size of this state */
} af8_small_state;

/* One tensor of a factored launch: a rows x cols matrix (row-major) or, with batch_rows > 0, a batch of
 * rows / batch_rows matrices of batch_rows x cols one after another (a tensor of more than two dimensions,
 * factored over its last two: optimizer.py:2203-2207).  For a batch the row arrays (row_sum, inv_row*, the row
 * states) still hold `rows` values, the column arrays (col_sum, inv_col*, the column states) hold
 * (rows / batch_rows) * cols values, matrix after matrix, and the mean that normalises the row factor is
 * taken per matrix.  Batches run through the general kernels: launch them with cfg.aligned8 = 0. */
typedef struct af8_factored_tensor {
    void *param;                /* rows*cols elements of cfg.param_dtype */
    const void *grad;           /* fp32 or bf16 */
    uint8_t *m_q;               /* momentum codes over the flattened tensor, or NULL */
    float *m_scale;
    float *m_f32;               /* fp32 momentum, or NULL */
    double *row_sum;            /* rows doubles: scratch, filled by af8_factored_stats */
    double *col_sum;            /* cols doubles: scratch */
    float *inv_row;             /* rows floats: rsqrt(row_var / mean) of the second moment */
    float *inv_col;             /* cols floats: rsqrt(col_var) */
    float *inv_row_conf;        /* CAME: the same for the confidence states */
    float *inv_col_conf;
    af8_small_state row_var, col_var;      /* second-moment states */
    af8_small_state conf_row, conf_col;    /* CAME confidence states */
    int64_t rows, cols;
    int64_t first_chunk;        /* running sum of ceil(rows*cols / chunk) (update passes) */
    int64_t first_tile;         /* running sum of stat tiles (af8_factored_stats): per matrix
                                   ceil(its rows / af8_factored_tile_rows()) * ceil(cols / af8_factored_tile_cols()) */
    float decay;                /* 1 - wd_mult*wd, 1.0 without weight decay */
    float alpha;
    float v_w;                  /* second-moment EMA weight beta_val */
    float m_w;                  /* float(1 - beta1) */
    float c_w;                  /* float(1 - beta3) */
    float eps1;
    float eps_came;
    int32_t first_small;        /* running sum of ceil(rows / B) + ceil(column values / B), B = row_var.block: this
                                   tensor's first unit in af8_factored_small (its row blocks, then its column blocks) */
    uint64_t sr_base;           /* stochastic rounding counter origin, as af8_fullrank_tensor.sr_base;
                                   element r*cols + c draws from counter sr_base + r*cols + c */
    void *param_copy;           /* optional bf16 copy of the updated fp32 parameter, as af8_fullrank_tensor.param_copy */
    int64_t batch_rows;         /* 0: one matrix; else the rows of one matrix of the batch (divides rows) */
} af8_factored_tensor;

enum {
    AF8_FSTAT_GRADSQ = 0,     /* row / column sums of g*g (optimizer.py:2221-2223) */
    AF8_FSTAT_RESIDUAL = 1    /* CAME: sums of (U - M)^2 + eps_came (optimizer.py:932-934) */
};

enum {
    AF8_FUPD_SUMSQ_U = 0,     /* per-chunk sum of squares of U = g*inv_row*inv_col (CAME clip,
                                 optimizer.py:826-828) or of the final update (d-clip / Fira) */
    AF8_FUPD_SUMSQ = 1,       /* per-chunk sum of squares of the final update */
    AF8_FUPD_APPLY = 2,       /* write parameters (and momentum codes), scaled by af8_dyn_scalars */
    AF8_FUPD_LAG = 3          /* APPLY with the scalars af8_lag_scalars(phase 0) prepared, plus this step's
                                 partial sums of squares of the raw update (lag_norm=True; not with CAME) */
};

typedef struct af8_factored_cfg {
    int32_t param_dtype;    /* AF8_F32, AF8_BF16 or AF8_F16 (rounding rules as in af8_fullrank_cfg) */
    int32_t grad_dtype;     /* AF8_F32, AF8_BF16 or AF8_F16 */
    int32_t m_fmt;          /* AF8_M_*; AF8_M_NONE when beta1 is None */
    int32_t m_block;
    int32_t came;           /* 1: CAME (needs momentum) */
    int32_t negate_grad;
    int32_t mode;           /* AF8_FSTAT_* for af8_factored_stats, AF8_FUPD_* for af8_factored_update */
    float v_floor;          /* min_log floor of the AL requantisation (-126) */
    int32_t aligned8;       /* 1: every tensor has cols % 8 == 0 and 16-byte aligned arrays
                               (checked by af8_factored_upload); selects the 128-bit kernels */
    int32_t stochastic_round; /* as af8_fullrank_cfg.stochastic_round */
    int64_t total_tiles;    /* optional: the table's number of statistic tiles (the last tensor's first_tile plus its
                               own tiles).  With it the sum-of-squares passes that only read the gradient
                               (AF8_FUPD_SUMSQ_U, AF8_FUPD_SUMSQ without momentum) run over the tiles, with the column
                               factors in registers; 0: over the flat chunks */
    int32_t cols_mult256;   /* 1: every tensor of the table has cols % 256 == 0 (with total_tiles: the write pass with a
                               UF8 momentum then also runs over the tiles, a row slice being one momentum block) */
    int32_t reserved;
} af8_factored_cfg;

/* Number of flattened elements per work unit of af8_factored_update for a
 * momentum block size (a multiple of m_block, at most 2048). */
AF8_API int32_t af8_factored_chunk(int32_t m_block);
/* Rows and columns per tile of af8_factored_stats. */
AF8_API int32_t af8_factored_tile_rows(void);
AF8_API int32_t af8_factored_tile_cols(void);

/* Validate a host table and copy it to the device (as af8_fullrank_upload). */
AF8_API int af8_factored_upload(const af8_factored_cfg *cfg, const af8_factored_tensor *host_tensors,
                                af8_factored_tensor *dev_tensors, int32_t n_tensors, void *stream);

/* Row and column sums in binary64 for every tensor: zeroes row_sum / col_sum,
 * then accumulates.  RESIDUAL mode reads dyn[i].pre_div (the clip divisor of U).
 * Replaces compute_factored_sums (kernels.cu:1946-1956) and fused_came_pass1
 * (kernels.cu:2223-2242). */
AF8_API int af8_factored_stats(const af8_factored_cfg *cfg, const af8_factored_tensor *dev_tensors,
                               const af8_factored_tensor *host_tensors, int32_t n_tensors,
                               const af8_dyn_scalars *dyn, void *stream);
/* The same with room for two tensor maps (128 bytes each) per tensor: host_maps is pinned, 64-byte aligned and
 * stays unchanged until its copy has run; dev_maps is device memory, 64-byte aligned.  In RESIDUAL mode over bf16
 * gradients and a UF8 momentum of block 256 with cfg.cols_mult256 set, the library describes every tensor's
 * gradient and momentum codes as [rows][cols] arrays for tiled bulk tensor copies (TMA) and the kernel brings
 * four rows of a 256-column slice in per copy instead of one.  Otherwise, or with NULL maps, it is
 * af8_factored_stats. */
AF8_API int af8_factored_stats_boxes(const af8_factored_cfg *cfg, const af8_factored_tensor *dev_tensors,
                                     const af8_factored_tensor *host_tensors, int32_t n_tensors,
                                     const af8_dyn_scalars *dyn, void *host_maps, void *dev_maps, void *stream);

/* Per tensor: means from the sums, EMA into the row / column states (second
 * moment when conf == 0, CAME confidence when conf != 0), requantisation, and
 * the inverse-std vectors inv_row / inv_col (or inv_*_conf).  Two launches: one CTA per
 * quantisation block of a state (total_units of them, see af8_factored_tensor.first_small), then
 * the mean of the row state and the inverse-std vectors.  The row sums are consumed: the first
 * entry of each block of row_sum is overwritten with the block's partial sum of the new state.
 * Replaces fused_log_quantize_lerp on the small states and the torch glue
 * around it (optimizer.py:2226-2252, 2289-2294, 818-821). */
AF8_API int af8_factored_small(const af8_factored_cfg *cfg, const af8_factored_tensor *dev_tensors,
                               int32_t n_tensors, int32_t conf, int32_t total_units, void *stream);

/* One pass over all elements in chunks.  block_sumsq: one DOUBLE per chunk
 * (SUMSQ modes; set af8_norm_tensor.partials_f64 when finalising them).  dyn: per-tensor scalars (pre_div always read when cfg->came,
 * step / fira / zero in APPLY mode).
 * Replaces fused_update_2d_*, compute_ut_rms and fused_came_pass2*
 * (kernels.cu:1651-1917, 1986-2000, 2244-2405). */
AF8_API int af8_factored_update(const af8_factored_cfg *cfg, const af8_factored_tensor *dev_tensors,
                                int32_t n_tensors, int64_t total_chunks, const af8_dyn_scalars *dyn,
                                double *block_sumsq, void *stream);

/* ------------------------------------------------------------------------ */
/* APOLLO: low-rank projected statistics                                     */
/* ------------------------------------------------------------------------ */

/* Host scalars of one tensor's APOLLO step (optimizer.py:2990-3023). */
typedef struct af8_apollo_scalars_in {
    float alpha;            /* alpha_t */
    float bc;               /* float(sqrt(bc2)/bc1) (bc_mode 1) or float(bc1) (bc_mode 2) */
    float d;                /* clip threshold, 0 disables */
    float clip_div;         /* float(sqrt(numel)*d) */
    float fira_margin1;     /* float(1 + fira_margin) */
    float sqrt_scale;       /* float(sqrt(apollo_scale)) */
    int32_t bc_mode;        /* 0 none, 1 multiply, 2 divide */
    int32_t fira;           /* enable_fira_for_apollo */
    int32_t fira_has_prev;  /* 0 on the tensor's first limited step */
    int32_t scale_tensor;   /* apollo_scale_type == "tensor" */
    int32_t scale_front;    /* apollo_scale_front */
    int32_t reserved;
} af8_apollo_scalars_in;

/* Device scalars produced by af8_apollo_scales and consumed by af8_apollo_apply. */
typedef struct af8_apollo_scalars {
    float update_scale;     /* -alpha/denom with bias correction */
    float fira;             /* Fira scale */
    float norm;             /* the global norm that was limited */
    float decay;            /* weight-decay factor when it was computed on the device (alpha_decay), else 1 */
} af8_apollo_scalars;

/* g_low = G @ Pt (rows >= cols; Pt is cols x rank, g_low rows x rank) or Pt @ G
 * (Pt is rank x rows, g_low rank x cols), every output being the correctly
 * rounded dot product, and chan_g2 = squared norm of every channel of G (rows
 * when rows >= cols, else columns) in binary64.  Non-finite gradient entries
 * count as zero (optimizer.py:2606).
 * Replaces torch.matmul (optimizer.py:2678-2681) and the channel norms
 * (optimizer.py:2975-2979). */
AF8_API int af8_apollo_project(const void *grad, int32_t grad_dtype, int32_t negate, const float *pt,
                               int64_t rows, int64_t cols, int64_t rank, float *g_low, double *chan_g2,
                               void *stream);

/* The same projection with a caller-provided workspace of at least
 * af8_apollo_project_workspace(rows, cols, rank) bytes, 256-byte aligned.  With bf16
 * gradients and rows, cols and rank multiples of 8 the contraction runs on the tensor
 * cores: Pt is split into three bf16 planes (exact to 24 bits) and accumulated in
 * binary32, i.e. the accuracy of an fp32 matmul instead of the correctly rounded dot
 * products of af8_apollo_project.  Any other case takes the exact path and ignores the
 * workspace.  Replaces torch.matmul (optimizer.py:2678-2681). */
AF8_API int64_t af8_apollo_project_workspace(int64_t rows, int64_t cols, int64_t rank);
AF8_API int af8_apollo_project_ws(const void *grad, int32_t grad_dtype, int32_t negate, const float *pt,
                                  int64_t rows, int64_t cols, int64_t rank, float *g_low, double *chan_g2,
                                  void *workspace, int64_t workspace_bytes, void *stream);

/* Many projections in one call.  Every descriptor that qualifies for the tensor-core path
 * (see af8_apollo_project_ws) joins ONE launch over the tiles of all tensors, which keeps
 * the GPU full when a single matrix has fewer tiles than there are SMs; the others take
 * the exact path one by one.  host_scratch (pinned, valid until the copies have run) and
 * dev_scratch each hold n * af8_apollo_project_task_bytes() bytes, 64-byte aligned.
 * transpose_scratch (device, 256-byte aligned, may be NULL with transpose_bytes 0) lets
 * left-case tensors (rows < cols) use the tcgen05 kernel, which wants both operands with the
 * contracted dimension contiguous: their gradients are transposed into it, as many tensors at
 * a time as fit; a tensor whose transposed gradient does not fit stays on the mma.sync kernel. */
typedef struct af8_apollo_proj_desc {
    const void *grad;       /* rows x cols */
    const float *pt;        /* cols x rank (rows >= cols) or rank x rows */
    float *g_low;           /* rows x rank or rank x cols */
    double *chan_g2;        /* max(rows, cols) */
    void *workspace;        /* af8_apollo_project_workspace() bytes, 256-byte aligned; NULL: exact path */
    int64_t workspace_bytes;
    int64_t rows, cols, rank;
    int32_t negate;
    int32_t planes_valid;   /* 1: the workspace still holds the bf16 planes of this same pt from an earlier call
                               (the projection matrix changes every apollo_update_proj_gap steps only): they are
                               not rebuilt */
} af8_apollo_proj_desc;
AF8_API int32_t af8_apollo_project_task_bytes(void);
AF8_API int af8_apollo_project_batch(const af8_apollo_proj_desc *descs, int32_t n, int32_t grad_dtype,
                                     void *host_scratch, void *dev_scratch, void *transpose_scratch,
                                     int64_t transpose_bytes, void *stream);

/* Scaling factors sf[channel] = ||update_low|| / (||g_low|| + 1e-8) (one entry
 * for the tensor-wide variant), the global norm, the Fira limiter, the clip
 * and the bias correction.  sums: 3 doubles of scratch.  fira_prev: device
 * scalar of the state key "scaled_grad_norm_prev".  alpha_decay: as
 * af8_apollo_finish_tensor.alpha_decay, or NULL.
 * Replaces compute_apollo_norms (kernels.cu:2441-2453), fira_scalar and the
 * torch glue of optimizer.py:2961-3023. */
AF8_API int af8_apollo_scales(const float *upd, const float *g_low, const double *chan_g2, int64_t rows,
                              int64_t cols, int64_t rank, const af8_apollo_scalars_in *in, float *sf,
                              double *sums, float *fira_prev, af8_apollo_scalars *out, const float *alpha_decay,
                              void *stream);

/* p = p*decay + (update_scale * G) * (sf[channel] * fira * sqrt_scale) for fp32
 * parameters.  Replaces the apollo_apply_* kernels (kernels.cu:2834-3000) and the
 * torch mul_/addcmul_ write-back (optimizer.py:3073-3079). */
/* af8_apollo_scales for all tensors of a group in two launches (channel-wise scaling only).
 * host_tensors is pinned and stays valid until the copy has run; dev_tensors holds n entries.
 * first_unit numbers 8-channel units across the table, total_units is their count. */
typedef struct af8_apollo_finish_tensor {
    const float *upd;       /* update_low, shaped like g_low */
    const float *g_low;
    const double *chan_g2;  /* from af8_apollo_project* */
    float *sf;              /* out: max(rows, cols) scaling factors */
    double *sums;           /* 3 accumulators */
    float *fira_prev;       /* limiter state (NULL without the limiter) */
    af8_apollo_scalars *out;
    int64_t rows, cols, rank;
    int64_t first_unit;
    af8_apollo_scalars_in in;
    const float *alpha_decay;   /* optional device pair {alpha_t, decay factor} written by af8_param_scale for
                                   scale_parameter=True (optimizer.py:850-853, 3007-3013): replaces in.alpha, and the
                                   decay factor is handed on in af8_apollo_scalars.decay; NULL: in.alpha */
} af8_apollo_finish_tensor;
AF8_API int af8_apollo_scales_batch(const af8_apollo_finish_tensor *host_tensors, af8_apollo_finish_tensor *dev_tensors,
                                    int32_t n, int64_t total_units, void *stream);

/* param_dtype AF8_F32, AF8_BF16 or AF8_F16.  A 16-bit parameter is rounded to nearest after the decay and
 * after the update, or, with stochastic_round, p*decay + (g*final_scale)*update_scale is formed in binary32
 * and rounded stochastically with the counter generator at sr_base (see af8_fullrank_tensor.sr_base;
 * optimizer.py:3043-3079, apollo_apply_{bf16,fp16}_{sr,det}).
 * param_copy: optional bf16 copy of the updated fp32 parameter (rows*cols 16-bit words, 16-byte aligned),
 * as af8_fullrank_tensor.param_copy; NULL for none.
 * has_decay: 0 none, 1 multiply by `decay`, 2 multiply by scalars->decay (computed on the device). */
AF8_API int af8_apollo_apply(void *param, int32_t param_dtype, int32_t stochastic_round, uint64_t sr_base,
                             const void *grad, int32_t grad_dtype, int32_t negate, const float *sf,
                             const af8_apollo_scalars *scalars, int64_t rows, int64_t cols,
                             const af8_apollo_scalars_in *in, float decay, int32_t has_decay, void *param_copy,
                             void *stream);

/* af8_apollo_apply for all tensors of a group in one launch (the reference writes back tensor by tensor,
 * optimizer.py:3043-3079; one launch keeps the memory system busy across the tensors' ends).  Every field as
 * the argument of the same name of af8_apollo_apply; scale_tensor, fira, scale_front and sqrt_scale as in
 * af8_apollo_scalars_in.  first_chunk numbers 2048-element chunks across the table, ceil(rows*cols / 2048)
 * per tensor, and total_chunks is their count.  host_tensors is pinned and stays valid until the copy has
 * run; dev_tensors holds n entries.  A table with a tensor that the 128-bit path cannot take (cols % 8 != 0,
 * an unaligned array, 2^34 elements or more) is applied tensor by tensor through af8_apollo_apply. */
typedef struct af8_apollo_apply_tensor {
    void *param;
    const void *grad;
    const float *sf;
    const af8_apollo_scalars *scalars;
    void *param_copy;           /* NULL for none */
    int64_t rows, cols;
    int64_t first_chunk;
    uint64_t sr_base;
    float sqrt_scale, decay;
    int32_t scale_tensor, fira, scale_front, has_decay, stochastic_round, reserved;
} af8_apollo_apply_tensor;
AF8_API int af8_apollo_apply_batch(const af8_apollo_apply_tensor *host_tensors, af8_apollo_apply_tensor *dev_tensors,
                                   int32_t n, int64_t total_chunks, int32_t param_dtype, int32_t grad_dtype,
                                   int32_t negate, void *stream);

/* ------------------------------------------------------------------------ */
/* APOLLO: further low-rank state rules                                      */
/* ------------------------------------------------------------------------ */

/* An AL-coded (q / scale / min_log) or fp32 state of n values. */
typedef struct af8_apollo_rule_state {
    void *q;            /* uint8 (AL8) / uint16 (AL16) codes, padded to the block; NULL for fp32 */
    float *scale;
    float *min_log;
    float *f32;         /* fp32 state when fmt == AF8_V_FP32 */
    int64_t n;
    int32_t fmt;        /* AF8_V_* */
    int32_t reserved;
} af8_apollo_rule_state;

/* update_low of one tensor under apollo_factorize and / or CAME (beta3), from the projected
 * gradient that af8_apollo_project* produced.  Replaces the corresponding branches of
 * _update_param_apollo (optimizer.py:2688-2760 factorised second moment, 2708-2750 its CAME form,
 * 2801-2903 CAME over the projected gradient; the arithmetic of the pure-PyTorch branches) and the
 * kernels compute_apollo_came_rms / apollo_came_compute_m_res / apollo_came_compute_update_norms
 * (kernels.cu:2455-2566).  The plain rule (neither flag) runs through af8_fullrank_step.
 * lr_rows x lr_cols is the projected shape: (rows, rank) when rows >= cols, else (rank, cols). */
typedef struct af8_apollo_rule {
    const float *g_low;         /* lr_rows * lr_cols */
    float *upd;                 /* out: update_low */
    void *work;                 /* af8_apollo_rule_workspace(lr_rows, lr_cols) bytes, 256-byte aligned */
    int64_t work_bytes;
    int64_t lr_rows, lr_cols;
    int32_t factorize;          /* apollo_factorize */
    int32_t came;               /* beta3 is not None (needs a momentum) */
    int32_t m_fmt;              /* AF8_M_*; AF8_M_NONE when beta1 is None */
    int32_t m_block;
    int32_t block;              /* AL block of v_low / res_low / conf_*_low */
    int32_t first_factor;       /* factorize: row_var_low / col_var_low hold no history yet (optimizer.py:2695) */
    int32_t first_v;            /* CAME without factorize: v_low holds no history yet (optimizer.py:2763) */
    int32_t reserved;
    float v_w;                  /* beta_val */
    float v_keep;               /* float(1 - beta_val) */
    float m_w;                  /* float(1 - beta1) */
    float c_w;                  /* float(1 - beta3) */
    float eps_came;
    float eps_sq;               /* max(apollo_eps^2, FLT_MIN) */
    float apollo_eps;
    float d;                    /* clip threshold of the low-rank U_t; <= 0: none */
    float v_floor_later;        /* log2(eps_sq): min_log floor of v_low after its first step */
    float reserved2;
    float *row_var_low;         /* factorize: fp32 [lr_rows] */
    float *col_var_low;         /* factorize: fp32 [lr_cols] */
    uint8_t *m_q;               /* momentum of the projected space: codes ... */
    float *m_scale;
    float *m_f32;               /* ... or fp32 */
    af8_apollo_rule_state v;            /* CAME without factorize: v_low, n = lr_rows * lr_cols */
    af8_apollo_rule_state res;          /* CAME without factorize: res_low, n = lr_rows * lr_cols */
    af8_apollo_rule_state conf_row;     /* factorize + CAME: conf_row_low, n = lr_rows */
    af8_apollo_rule_state conf_col;     /* factorize + CAME: conf_col_low, n = lr_cols */
} af8_apollo_rule;

AF8_API int64_t af8_apollo_rule_workspace(int64_t lr_rows, int64_t lr_cols);
/* rule: HOST pointer.  Everything runs on `stream`; no host synchronisation. */
AF8_API int af8_apollo_rule_step(const af8_apollo_rule *rule, void *stream);

/* ------------------------------------------------------------------------ */
/* Step without caller-provided working memory                               */
/* ------------------------------------------------------------------------ */

/* The limited full-rank step (statistic pass, norm / Fira / clip scalars, apply
 * pass) for ONE tensor, using no memory besides the tensor's own parameter,
 * gradient and states.  It has no counterpart in the reference.
 *
 * It exists for callers that cannot come up with device buffers when they
 * step: a foreign-language binding that only forwards pointers it was given
 * and has no device allocator, or a process in which a framework's allocator
 * already holds the whole GPU, so that an extra cudaMalloc would fail or stall.
 * The descriptor row, the per-tensor scalars and the per-block partial sums
 * that af8_fullrank_step takes from the caller live here in a 1 MiB array that
 * is part of the library image (each GPU that loads the library holds one copy
 * until the process ends).  The call performs no cudaMalloc / cudaFree and uses
 * no allocating library routine.
 *
 *   cfg          as for af8_fullrank_step; cfg->mode is ignored and the
 *                momentum-only rule is not covered
 *   host_tensor  HOST pointer to one filled af8_fullrank_tensor (first_block is
 *                ignored); passed to the device as a kernel argument
 *   clip_d       RMS clip threshold d (0 disables)
 *   fira         non-zero: run the Fira norm-growth limiter with fira_margin1 =
 *                float(1 + fira_margin); fira_prev is the device scalar that holds the previous limited
 *                norm (read when fira_has_prev != 0, always written)
 *   norm_out     optional device float that receives the measured update norm
 *
 * Limit: at most af8_noalloc_max_numel(cfg->block) elements (262,080 V blocks:
 * 536,739,840 elements at block 2048); larger tensors are rejected with
 * AF8_ERR_UNSUPPORTED and a message that names the limit.
 *
 * The first call on each device resolves the array's device address (which can
 * load the library's device code); make that first call outside any stream
 * capture.  All calls on a device share the one array and it keeps the previous
 * call's contents; the call itself clears what it needs cleared.  Two calls
 * whose GPU work can overlap (different streams, different threads) race on
 * the array: serialise them on one stream or with events. */
AF8_API int af8_fullrank_limited_step_noalloc(const af8_fullrank_cfg *cfg,
                                              const af8_fullrank_tensor *host_tensor,
                                              float clip_d, int32_t fira, float fira_margin1,
                                              float *fira_prev, int32_t fira_has_prev,
                                              float *norm_out, void *stream);

/* Largest tensor the call above accepts for a V block size (0 for an invalid
 * block size). */
AF8_API int64_t af8_noalloc_max_numel(int32_t block);

/* ------------------------------------------------------------------------ */
/* Parameter-scaled step size                                                */
/* ------------------------------------------------------------------------ */

/* One tensor of af8_param_scale. */
typedef struct af8_scale_tensor {
    const void *param;          /* numel elements of param_dtype */
    int64_t numel;
    int64_t first_chunk;        /* running sum of ceil(numel / af8_scale_chunk()) */
    float sqrt_n;               /* float(sqrt(numel)) */
    float rho;                  /* relative or fixed learning rate of this step */
    float eps2;                 /* lower bound of the parameter RMS */
    float bc;                   /* bias-correction factor, see bc_mode */
    float weight_decay;         /* 0 disables */
    int32_t bc_mode;            /* 0: none, 1: alpha *= bc, 2: alpha /= bc */
    int32_t scale_weight_decay; /* 1: decay uses alpha, 0: decay uses rho */
    int32_t param_dtype;        /* AF8_F32, AF8_BF16 or AF8_F16 */
    const double *total;        /* when not NULL: device location of the whole tensor's sum of squares, used by
                                   af8_param_scale_finish instead of this table entry's partial sums (a tensor
                                   spread over several tables or GPUs; sqrt_n then describes the whole tensor) */
} af8_scale_tensor;

/* alpha = max(||p|| / sqrt(n), eps2) * rho (then bias correction) and
 * decay = 1 - mult * weight_decay for every tensor, written into the float
 * fields at alpha_offset / decay_offset of row i of a device table whose rows
 * are table_stride bytes apart (for af8_fullrank_tensor: its size, and the offsets of
 * `alpha` and `decay`).  chunk_sumsq is scratch: one float per chunk of
 * af8_scale_chunk() parameters, summed over the tensors.
 * Replaces the torch.linalg.vector_norm pass of _compute_alpha with
 * scale_parameter=True (optimizer.py:850-853) and the 0-d tensor arithmetic
 * after it (optimizer.py:2020-2039). */
AF8_API int af8_param_scale(const af8_scale_tensor *host_tensors,
                            af8_scale_tensor *dev_tensors, int32_t n_tensors,
                            float *chunk_sumsq, void *dev_table, int64_t table_stride,
                            int64_t alpha_offset, int64_t decay_offset, void *stream);

/* The two halves of af8_param_scale, for callers that must combine partial sums between them (a tensor
 * spread over several GPUs: sum the tensor's entries of chunk_sumsq, all-reduce, point
 * af8_scale_tensor.total at the result).  af8_param_sumsq validates and uploads the table and fills
 * chunk_sumsq; af8_param_scale_finish evaluates alpha / decay from the device table left by it.
 * No counterpart in the reference (single-GPU). */
AF8_API int af8_param_sumsq(const af8_scale_tensor *host_tensors, af8_scale_tensor *dev_tensors,
                            int32_t n_tensors, float *chunk_sumsq, void *stream);
AF8_API int af8_param_scale_finish(const af8_scale_tensor *dev_tensors, int32_t n_tensors,
                                   const float *chunk_sumsq, void *dev_table, int64_t table_stride,
                                   int64_t alpha_offset, int64_t decay_offset, void *stream);

/* Number of parameters per partial sum of af8_param_scale. */
AF8_API int af8_scale_chunk(void);

/* ------------------------------------------------------------------------ */
/* Stand-alone codecs (state migration, checkpoint conversion, tests)        */
/* ------------------------------------------------------------------------ */

/* AL8/AL16 -> fp32.  Replaces dequantize_log_nonneg (kernels.cu:2613-2632). */
AF8_API int af8_al_dequant(const void *q, const float *scale, const float *min_log,
                   int64_t numel, int32_t block, int32_t bits, float *out,
                   void *stream);

/* fp32 -> AL8/AL16 with fresh per-block ranges; q holds ceil(numel/block)*block
 * codes.  Replaces the quantise half of fused_log_quantize_lerp
 * (kernels.cu:482-517) and _log_quantize_nonneg (optimizer.py:299-325). */
AF8_API int af8_al_quant(const float *x, int64_t numel, int32_t block, int32_t bits,
                 float floor_log, void *q, float *scale, float *min_log,
                 void *stream);

/* momentum codes -> fp32.  Replaces dequantize_dynamic (kernels.cu:2585-2590)
 * and _dequantize_uniform_pytorch (optimizer.py:522-532). */
AF8_API int af8_m_dequant(const uint8_t *q, const float *scale, int64_t numel,
                  int32_t m_block, int32_t m_fmt, float *out, void *stream);

/* fp32 -> momentum codes.  Replaces the quantise half of
 * fused_m_quantize_lerp (kernels.cu:574-588) and _m_quantize
 * (optimizer.py:547-552). */
AF8_API int af8_m_quant(const float *m, int64_t numel, int32_t m_block, int32_t m_fmt,
                uint8_t *q, float *scale, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* AF8_H */
