/*
 * zgml_cuda.h — C-ABI of the B200 (sm_100a) CUDA backend for zgml's
 * DeviceProgram interface.
 *
 * This is the drop-in boundary.  A thin `src/backend/cuda.zig` (see
 * zig/cuda.zig and INTEGRATION.md) flattens zgml's Zig slices / tagged unions
 * into the PODs below and forwards the six `Backend.VTable` slots
 * (reference src/backend.zig:339-352) to the `zg_cuda_*` entry points, exactly
 * as src/backend/metal.zig wraps src/backend/metal_shim.h.
 *
 * Plain pointers and sizes only; no C++ / torch types.  All offsets and strides
 * are in f32 ELEMENTS unless a field says bytes (ZgIO is bytes, like ProgramIO).
 */
#ifndef ZGML_CUDA_H
#define ZGML_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ── zgml `Op` ordinals (reference src/op.zig:11-61, declaration order) ───── */
enum {
    ZG_EW_NONE = 0, ZG_EW_VIEW = 1, ZG_EW_RESHAPE = 2, ZG_EW_TRANSPOSE = 3,
    ZG_EW_PERMUTE = 4, ZG_EW_AS_STRIDED = 5, ZG_EW_BROADCAST_TO = 6,
    ZG_EW_ADD = 7, ZG_EW_MUL = 8,
    ZG_EW_NEG = 9, ZG_EW_ABS = 10, ZG_EW_SGN = 11, ZG_EW_STEP = 12, ZG_EW_RELU = 13,
    ZG_EW_SQRT = 14, ZG_EW_RECIP = 15, ZG_EW_EXP = 16, ZG_EW_LOG = 17, ZG_EW_GELU = 18,
    ZG_EW_SUM = 19, ZG_EW_MAX = 20, ZG_EW_REPEAT = 21
};

/* ── DeviceOp tags (reference src/backend.zig:179-249, union field order) ─── */
typedef enum ZgOpTag {
    ZG_OP_ELEMENTWISE = 0,
    ZG_OP_MATMUL = 1,
    ZG_OP_QMATMUL = 2,
    ZG_OP_SOFTMAX = 3,
    ZG_OP_LAYERNORM = 4,
    ZG_OP_RMSNORM = 5,
    ZG_OP_REDUCE = 6,
    ZG_OP_REPEAT = 7,
    ZG_OP_SLICE_ASSIGN = 8,
    ZG_OP_ROPE = 9,
    ZG_OP_ATTENTION = 10,
    ZG_OP_FUSED_ELEMENTWISE = 11,
    ZG_OP_COUNT = 12,
    /* Extensions (no zgml counterpart: the reference has no distributed layer).  Emitted only by
     * the sharded session of this repo; need zg_cuda_comm_init().  One NCCL collective each, in program order. */
    ZG_OP_ALLREDUCE = 12, /* buf[offset .. offset + n) = sum over ranks, in place */
    ZG_OP_ALLGATHER = 13, /* dst[dst_offset + r * n ..) = rank r's src[src_offset .. + n), every rank */
    /* Sequence-model extensions (no zgml counterpart): the building blocks of decoder stacks that are not LLaMA-shaped —
     * dense 16-bit / f32 weights, affine norms with a fused residual, windowed attention with a sink, short causal
     * convolutions, a gated delta-rule recurrence, a routed mixture of experts; and (from TOKEN_SHIFT on) mixers that
     * attend over a per-sequence cache of keys and values or of one latent that serves as both: token shift, a learned
     * average over the depth of the stack, rotary positions, the cache append, attention over the cache with grouped heads,
     * several score maps per head and causal / window / block masks, head-wise products, PolyNorm.  All take a ZgSeqOp
     * (below); per-sequence state (key ring or cache, recurrent state, convolution tail, shifted row) lives in EXTERNAL
     * buffers shared by the programs of a session,
     * and the run-time position / state slot / token ids are read from a small control buffer, so one CUDA graph serves
     * every step. */
    ZG_OP_EMBED = 14,
    ZG_OP_LINEAR = 15,
    ZG_OP_NORM = 16,
    ZG_OP_WINDOW_ATTENTION = 17,
    ZG_OP_CAUSAL_CONV = 18,
    ZG_OP_DELTA_RULE = 19,
    ZG_OP_ROUTE = 20,
    ZG_OP_MOE_FFN = 21,
    ZG_OP_TOKEN_SHIFT = 22,
    ZG_OP_DEPTH_MIX = 23,
    ZG_OP_ROTARY = 24,
    ZG_OP_CACHE_APPEND = 25,
    ZG_OP_CACHED_ATTENTION = 26,
    ZG_OP_MAP_COMBINE = 27,
    ZG_OP_GATE = 28,
    ZG_OP_HEAD_LINEAR = 29,
    ZG_OP_POLY_NORM = 30,
    /* Recurrent mixers with an elementwise or scalar decay, and what surrounds them (csrc/recops.cu): the state-space scan
     * of Mamba-2, the minimal gated recurrent unit, a gated group norm, a per-head RMS norm with a position-dependent
     * query temperature, stand-alone activations, and the real-gated linear recurrent unit. */
    ZG_OP_SSM_SCAN = 31,
    ZG_OP_MIN_GRU = 32,
    ZG_OP_GATED_NORM = 33,
    ZG_OP_HEAD_NORM = 34,
    ZG_OP_ACTIVATION = 35,
    ZG_OP_RG_LRU = 36,
    ZG_OP_END = 37
} ZgOpTag;

/* Parameter pack of the sequence-model ops.  buf[] are program buffer indices (ZG_NO_BUF: absent), off[] element offsets,
 * n[] integers, f[] floats; buf[0] is always the destination.  Activations are f32.  A WEIGHT operand is (buffer, offset in
 * weight elements) plus the op's `wdt`: ZG_W_F32 (the buffer holds floats) or ZG_W_BF16 (it holds bfloat16 bit patterns,
 * two per f32 slot; widened exactly on load).  Linear weights are [out, in] row-major, applied as W x.  All arithmetic and
 * accumulation is f32.
 *
 * Control buffer `ctl` (int32 words inside an f32 buffer, written by the host before every execution):
 *   [0] position of the step's first token in its sequence, [1] state slot, [ZG_CTL_IDS ..) the step's token ids.
 *
 * EMBED             dst[t, :] = table[ids[t], :] * f0; with n3 = 1 a learned position row joins it, unscaled: + positions[p(t), :]
 *                   (a second table at off 1 of the same arena, p(t) = the token's position in its sequence)
 *                   buf 0 dst 1 ctl 2 table | off 0 table 1 positions | n 0 T 1 D 2 wdt 3 positions | f 0 scale
 * LINEAR            dst[m, n] = act(sum_k src[m, k] W[n, k] (+ bias[n])); act (n6): 0 none, 1 + the ACTIVATION kind otherwise (f0: its
 *                   parameter, where the kind has one)
 *                   buf 0 dst 1 src 2 W 3 bias 4 ctl | off 0 W 1 bias 2 src 3 dst | n 0 M 1 N 2 K 3 src row stride 4 dst row stride 5 wdt 6 act
 *                   7 source slot stride
 *                   With n7 > 0 the source rows are those of a per-sequence state buffer (a ring): n7 elements per slot, the slot
 *                   from the control buffer buf 4.
 *                   f 0 activation parameter
 * NORM              dst = (res +) norm(src) * w ; kind bit 0 clear: (x - mean) / sqrt(var + eps), set: x / sqrt(mean(x^2) + eps);
 *                   kind bit 1: the weight is stored around zero and applied as (1 + w); kind bit 2: the result is also
 *                   multiplied by the gain f1 (a scale of the following product folded into its input);
 *                   kind bit 3: Dynamic Tanh instead of a norm, tanh(alpha x) * w + b with no statistics of the row: the bias b
 *                   (cols values) and the scalar alpha follow w in its arena; kind bit 4: no norm and no weight, the row
 *                   itself (times the gain with bit 2): dst = res + gain * src, the plain residual step of a pre-norm stack.
 *                   Bits 3 and 4 combine with a residual and a chained norm, not with the averaged source or the token shift.
 *                   with n7 = 1 (kinds with statistics, no averaged source): buf 6 is a SECOND source, normed like the first with a
 *                   weight of its own (off 2 of w's arena) and added to it: dst = res + norm(src) w + norm(src2) w_b
 *                   with buf 4: also dst2 = norm(dst) * w2 in the same launch (the norm closing a sublayer and the one opening the next)
 *                   with buf 6 (single-row steps): the last output of the launch then passes a TOKEN_SHIFT (mix at off 2 of the
 *                   arena of the norm it follows, state buf 6, ctl buf 7) in the same launch
 *                   w and w2 must be constants of the model (an uploaded arena): they are read before the producing op of src has finished
 *                   with n 5 > 0 (no res, no chained norm): the row that is normed is the DEPTH_MIX of n5 streams of src (stride n6,
 *                   coefficients at off 4 of w's arena); buf 4 receives that average itself
 *                   buf 0 dst 1 src 2 w 3 res 4 dst2 5 w2 6 shift state 7 ctl | off 0 w 1 w2 2 shift mix 3 dst 4 average coefficients
 *                   n 0 rows 1 cols 2 kind 3 wdt 5 averaged streams 6 their stride 7 second source
 *                   4 kind of dst2 | f 0 eps 1 gain
 * WINDOW_ATTENTION  causal attention over the last `window` positions whose keys double as values (one projection, one cache),
 *                   grouped query heads, scores capped smoothly (cap * tanh(s / cap), f1 = 0: off), a per-distance per-head
 *                   additive bias table [window, H] (f32 program buffer), a softmax whose denominator carries an extra 1 (a
 *                   sink with score 0 and no value), and an elementwise sigmoid gate on the heads' output.  The step's keys
 *                   are first appended to a ring of R >= window - 1 + T positions per state slot (external buffer
 *                   [slots, R, G * dim]; position p lives in row p mod R).
 *                   buf 0 dst [T, H * dim] 1 proj (rows hold q | k | gate logits) 2 key ring 3 bias table 4 ctl
 *                   off 0 q 1 k 2 gate (columns inside a proj row) | n 0 T 1 H 2 G 3 dim 4 proj row stride 5 window 6 R
 *                   f 0 score scale 1 cap
 * CAUSAL_CONV       per-channel FIR over time with carried inputs: dst[t, c] = act(sum_j w[c, j] x[t - (taps - 1) + j, c]), x
 *                   before the step taken from the state (external [slots, taps - 1, C], zeros for a fresh slot), which is then
 *                   advanced by the step's inputs.  act 0: none, 1: SiLU.
 *                   With n7 = 1 a bias per channel (off 3 of w's arena) is added before the activation.
 *                   buf 0 dst 1 src 2 w [C, taps] 3 state 4 ctl | off 0 w 1 src 2 dst 3 bias | n 0 T 1 C 2 taps 3 src row stride
 *                   4 dst row stride 5 act 6 wdt 7 bias
 * DELTA_RULE        gated delta rule with one decay per head and key channel, state S [dim, vdim] per head (external
 *                   [slots, H, dim, vdim], f32): q, k -> unit vectors (x / sqrt(sum x^2 + f1)), q *= f2; beta = sigmoid(b);
 *                   g = exp(-exp(A_log[h]) * softplus(a + dt_bias)); per token S <- g * S (rows), u = beta * (v - S^T k),
 *                   S <- S + k u^T, o = S^T q; then o / sqrt(mean(o^2) + f0) * norm_w * sigmoid(gate).  Query / key head of
 *                   head h is h / (H / G).
 *                   buf 0 dst [T, H * vdim] 1 qkv 2 beta logits 3 a 4 gate logits 5 weights 6 state 7 ctl
 *                   off 0 q 1 k 2 v (columns of a qkv row) 3 beta (column of its row) 4 A_log 5 dt_bias 6 norm_w (weights)
 *                   7 gate (column of its row)
 *                   n 0 T 1 H 2 G 3 dim 4 vdim 5 qkv row stride 6 beta row stride 7 a row stride 8 gate row stride 9 wdt
 *                   10 form 11 dst row stride (0: H * vdim) 12 dst column
 *                   f 0 output-norm eps 1 unit-vector eps 2 q scale 3 decay temperature 4 output scale
 *                   Form bits (n10), all clear for the rule above.  Bit 0, plain accumulation (gated linear attention): no
 *                   unit vectors (q is only scaled by f2) and no correction by what the state already holds, u = v:
 *                   S <- g * S + k v^T, o = S^T q; buf 2 is not read.  Bit 1: the decay is g = sigmoid(a + dt_bias)^(1 / f3),
 *                   evaluated as exp(-softplus(-(a + dt_bias)) / f3); A_log is not read.  Bit 2: the output gate is
 *                   silu(gate) instead of sigmoid(gate).  Bit 3: the result is multiplied by f4.  It may land in columns of a
 *                   wider row (n11, n12), beside another mixer's heads.
 * ROUTE             mode 0: s = softmax(logits) over all NE outputs; the `top` largest of s + correction are chosen (ties:
 *                   lowest index); dst[t, c] = {index as int32 bits, s[index]} (weights not renormalised)
 *                   mode 1: z = logits + correction (a bias); the `top` largest z are chosen (ties: lowest index) and weighted
 *                   by the softmax over the chosen z alone
 *                   mode 2: s = sigmoid(logits); choice scores s + correction; the outputs form n6 equal groups of neighbours, a
 *                   group scores the sum of its two largest choice scores and only outputs of the n7 best groups can be chosen
 *                   (n6 <= 1: no groups); the `top` largest choice scores are chosen (ties: lowest index) and weighted by
 *                   their s divided by (the sum of the chosen s + 1e-20)
 *                   buf 0 dst [T, top, 2] 1 logits 2 correction | off 0 correction 1 logits | n 0 T 1 NE 2 top 3 logits row
 *                   stride 4 wdt 5 mode 6 groups 7 groups kept
 * MOE_FFN           dst[t] = sum_c weight_c * expert_{index_c}(src[t]); expert e < E: W_down (g * sigmoid(f1 * g) * (u + f2)),
 *                   g = min(W_gate x, f0), u = clamp(W_up x, -f0, f0); index >= E: the identity (x itself).  Expert weights
 *                   are stacked [E, ff, D] (gate, up) and [E, D, ff] (down).
 *                   buf 0 dst 1 src 2 route 3 weights 4 scratch [T, top, ff] | off 0 gate 1 up 2 down | n 0 T 1 D 2 ff 3 E
 *                   4 top 5 wdt | f 0 limit (INFINITY: none) 1 alpha 2 offset of the up branch
 * TOKEN_SHIFT       dst[t] = src[t] + (src[t - 1] - src[t]) * mix, element by element; src[-1] is the last row of the previous step
 *                   (state, external [slots, D], zeros for a fresh slot), and the state becomes src[T - 1].
 *                   buf 0 dst 1 src 2 mix 3 state 4 ctl | off 0 mix | n 0 T 1 D 2 wdt
 * DEPTH_MIX         dst[e] = sum_{j < terms} coeff[j] * hist[j * stride + e]: a learned average over the outputs of earlier layers
 *                   buf 0 dst 1 hist 2 coeff | off 0 coeff | n 0 elements 1 terms 2 stride 3 wdt
 * ROTARY            rotary positions on `heads` vectors per row, in place or (buf 2) read from another buffer: layout 0 pairs
 *                   (2i, 2i + 1), layout 1 pairs (i, i + dims / 2); pair i of the token at position p turns by
 *                   p * base^(-2i / dims), or, with buf 3, by p * table[i]: dims / 2 frequencies in f32 (any schedule: scaled,
 *                   blended, interpolated), in a buffer of the model at element off 2.  Angles in f32.
 *                   buf 0 x 1 ctl 2 src 3 frequency table | off 0 column of the first vector 1 its column in src 2 table offset
 *                   n 0 T 1 heads 2 head stride 3 row stride 4 dims 5 layout 6 src head stride 7 src row stride | f 0 base
 * CACHE_APPEND      the step's rows join a per-sequence cache (external [slots, R, width]; position p lives in row p mod R).
 *                   Of the appended columns the first `normed` are RMS-normed with a plain weight (a latent), the next `rot`
 *                   get the token's rotary position (a key part shared by all heads), the rest is copied.  With n9 > 0 the
 *                   normed columns are normed in groups of n9 (key heads), every group with the same weight of n9 values.
 *                   With off5 > 0 the same launch norms off5 QUERY heads of n9 values in place in the source rows (column off 3,
 *                   weight at off 4), times the temperature 1 + f2 * ln(floor((p + 1) / off6) + 1) (off6 = 0: none): HEAD_NORM fused.
 *                   With n10 > 0 (and n9 > 0) every normed group — key heads, and the query heads of off5 — is first turned by
 *                   the token's rotary position on its first n10 values (layout n8; frequencies base^(-2i / n10) from f1, or
 *                   from the f32 table buf 4 at element off 7, as ROTARY takes it), and the root mean square is that of the
 *                   turned vector: ROTARY fused, for designs that norm after the rotation.
 *                   buf 0 cache 1 src 2 ctl 3 norm weight 4 frequency table | off 0 src column 1 cache column 2 norm weight 3 query column
 *                   4 query weight 5 query heads 6 temperature period 7 frequency table offset
 *                   n 0 T 1 columns 2 src row stride 3 width 4 R 5 normed 6 rot 7 wdt 8 rotary layout 9 norm group 10 rotary inside the groups
 *                   f 0 eps 1 rotary base 2 temperature coefficient
 * CACHED_ATTENTION  softmax attention of the step's queries over cached keys and values.  A query row holds H * maps vectors
 *                   of dk (head h, map m at (h * maps + m) * dk); a key row G * maps vectors of dk; a value row G vectors of
 *                   dv; query (h, m) reads key (h / (H / G), m) and value h / (H / G).  The value cache may be the key cache
 *                   (a latent that serves as both).  Masks: 0 causal, 1 the last `size` positions, 2 causal inside blocks
 *                   of `size` positions counted from position 0.  R must cover what the mask can reach plus the step.
 *                   With buf 5 a score table [H * maps, off 6] (f32) indexed by the distance i - j is added to the scaled score
 *                   (any distance bias; a constant per head folds into it).  Weights (off 5): 0 softmax over the visible keys,
 *                   1 sigmoid(score) of every visible key, not normalised over the keys.
 *                   buf 0 dst [T, H * maps, dv] 1 q 2 key cache 3 value cache 4 ctl 5 score table
 *                   With f1 > 0 the scaled score is capped smoothly first: f1 * tanh(s / f1).  With buf 6 a learned SINK per
 *                   (head, map) joins the softmax: exp(sink) is added to the denominator alone; it has no key and no value, is
 *                   neither scaled nor capped, and counts once (a weight operand: element off 7 of buf 6, type n12).  The
 *                   result is multiplied by f2 where n13 = 1 and may land in columns of a wider row (n10 row stride, 0: H * maps * dv;
 *                   n11 first column), beside another mixer's heads.
 *                   buf 0 dst [T, H * maps, dv] 1 q 2 key cache 3 value cache 4 ctl 5 score table 6 sinks
 *                   off 0 q column 1 key column 2 value column (inside a cache row) 3 mask kind 4 mask size 5 weights 6 table row length
 *                   7 sinks
 *                   n 0 T 1 H 2 G 3 maps 4 dk 5 dv 6 q row stride 7 key row width 8 value row width 9 R 10 dst row stride
 *                   11 dst column 12 wdt of the sinks 13 output scale given 14 caches without slots (rows the program itself computed
 *                   for this step, position p in row p mod R as in a ring) | f 0 score scale 1 score cap 2 output scale
 * MAP_COMBINE       differential attention's combination of two maps: o = a[.., 0, :] - f0 * a[.., 1, :], then
 *                   o / sqrt(mean(o^2) + f1) * f2 per (token, head)
 *                   buf 0 dst [rows, dv] 1 src [rows, 2, dv] | n 0 rows 1 dv | f 0 lambda 1 eps 2 output scale
 * GATE              dst[t, c] *= sigmoid(gate[t, c / group]), in place (group = dv: one gate per head; 1: per element)
 *                   buf 0 dst 1 gate | off 0 gate column | n 0 T 1 columns 2 group 3 gate row stride 4 dst row stride
 * HEAD_LINEAR       a block-diagonal product: dst[t, h, n] = sum_k src[t, h, k] W[h, n, k], W stacked [H, N, K]; with buf 3 the
 *                   result is multiplied by sigmoid(gate[t, (h N + n) / group]) (the GATE op in the epilogue)
 *                   buf 0 dst 1 src 2 W 3 gate | off 0 W 1 src column 2 dst column 3 gate column 4 gate row stride
 *                   n 0 T 1 H 2 N 3 K 4 src head stride 5 src row stride 6 dst head stride 7 dst row stride 8 wdt 9 gate group
 * POLY_NORM         dst[t] = a N(z) + b N(z^2) + c N(z^3) + e with N(v) = v / sqrt(mean(v^2) + f0) over the row, powers taken
 *                   element by element, (a, b, c, e) four weights; may run in place
 *                   buf 0 dst 1 src 2 coefficients | off 0 coefficients | n 0 T 1 columns 2 wdt | f 0 eps
 * SSM_SCAN          state-space recurrence with one scalar decay per head and token (Mamba-2): dt = softplus(dt_logit + dt_bias[h]),
 *                   S <- exp(-exp(A_log[h]) dt) S + dt B x^T (S is N x P per head, f32), y = S^T C + D[h] x.  Head h reads the B and
 *                   C of group h / (H / G).  x | B | C are columns of one row (the output of the short convolution), the dt
 *                   logits columns of another.  The state is external [slots, zg_cuda_seq_state_elems(op)] in a layout private
 *                   to the op, zeros for a fresh slot.
 *                   buf 0 dst [T, H * P] 1 xbc 2 dt 3 weights 4 state 5 ctl
 *                   off 0 x 1 B 2 C (columns of an xbc row) 3 dt (column of its row) 4 A_log 5 dt_bias 6 D (weights)
 *                   n 0 T 1 H 2 G 3 N 4 P 5 xbc row stride 6 dt row stride 7 wdt
 * MIN_GRU           gated recurrence whose gates read the current token only: z = sigmoid(zl), c = u + 1/2 where u >= 0 and
 *                   sigmoid(u) where u < 0, S <- (1 - z) S + z c element by element (external [slots, W], zeros for a fresh
 *                   slot), dst = S * silu(g).  zl | u | g are columns of one row (biases belong to the projection).
 *                   buf 0 dst 1 proj 2 state 3 ctl | off 0 zl 1 u 2 g (columns) | n 0 T 1 W 2 proj row stride 3 dst row stride
 * GATED_NORM        dst = N(src * silu(gate)) * w with N an RMS norm over each of n2 equal parts of the row (the gate comes
 *                   before the norm); may run in place
 *                   buf 0 dst 1 src 2 gate 3 w | off 0 gate column 1 w | n 0 T 1 columns 2 groups 3 gate row stride 4 wdt
 *                   5 src row stride 6 dst row stride | f 0 eps
 * HEAD_NORM         per-head RMS norm in place with one weight of `dim` values shared by the heads, times a temperature that
 *                   grows with the position p of the token: 1 + f1 * ln(floor((p + 1) / n5) + 1) (n5 = 0: none)
 *                   buf 0 x 1 w 2 ctl | off 0 column of the first head 1 w | n 0 T 1 heads 2 dim 3 row stride 4 wdt 5 period
 *                   f 0 eps 1 temperature coefficient
 * ACTIVATION        dst = act(src) element by element, may run in place; kinds: 0 relu(z)^2, 1 silu, 2 gelu (tanh form), 3 relu,
 *                   4 smooth cap f0 * tanh(z / f0)
 *                   buf 0 dst 1 src | n 0 elements 1 kind | f 0 parameter of the kind
 * RG_LRU            real-gated linear recurrent unit, element by element over W channels: r = sigmoid(rl + r_bias),
 *                   i = sigmoid(il + i_bias), log a = -f0 * r * softplus(lam), S <- a S + sqrt(1 - a^2) (i u) (external
 *                   [slots, W], zeros for a fresh slot; the first token is no special case), dst = S * act(y) (n9: 0 the
 *                   column itself, 1 + the ACTIVATION kind otherwise).  The gate logits rl | il come from a block-diagonal
 *                   product: channel c lies at column (c / n4) * n5 + c % n4 of its row, from off 1 (rl) and off 2 (il).
 *                   buf 0 dst 1 u 2 gate logits 3 y 4 weights 5 state 6 ctl
 *                   off 0 u column 1 rl column 2 il column 3 y column 4 r_bias 5 i_bias 6 lam (weights)
 *                   n 0 T 1 W 2 u row stride 3 gate row stride 4 gate block width 5 gate block stride 6 y row stride
 *                   7 dst row stride 8 wdt 9 act of y | f 0 the constant in log a */
#define ZG_NO_BUF 0xFFFFFFFFu
#define ZG_W_F32 0
#define ZG_W_BF16 1
#define ZG_CTL_POS 0
#define ZG_CTL_SLOT 1
#define ZG_CTL_IDS 8
typedef struct ZgSeqOp {
    uint32_t buf[8];
    uint32_t off[8];
    uint32_t n[16];
    float f[8];
} ZgSeqOp;

/* MatMulGeometry — reference src/backend.zig:146-158 (all usize). */
typedef struct ZgMatMulGeometry {
    size_t M, N, K;
    size_t a_row_stride, a_col_stride;
    size_t b_row_stride, b_col_stride;
    size_t a_offset, b_offset, dst_offset, dst_row_stride;
} ZgMatMulGeometry;

/* FusedEwStep — reference src/backend.zig:170-175. */
typedef struct ZgFusedEwStep {
    uint32_t op;               /* ZG_EW_* */
    uint32_t is_swapped;       /* chain value sits in src1 position */
    uint32_t secondary_buf;    /* u16 in zgml */
    uint32_t secondary_offset;
} ZgFusedEwStep;

/* One DeviceOp.  Field names and meaning copied 1:1 from src/backend.zig:180-248;
 * u16 buffer indices are widened to u32. */
typedef struct ZgOp {
    uint32_t tag; /* ZgOpTag */
    uint32_t _pad;
    union {
        struct { uint32_t op, dst, src0, src1, n, dst_offset, src0_offset, src1_offset; } elementwise;
        struct { uint32_t dst, a, b, _pad; ZgMatMulGeometry geom; } matmul;
        struct {
            uint32_t dst, input, weight_idx, M, N, K;
            uint32_t input_offset, input_row_stride; /* stride 0 => K */
            uint32_t dst_offset, dst_row_stride;     /* stride 0 => N */
        } qmatmul;
        struct { uint32_t dst, src, rows, cols, src_offset, dst_offset; } softmax;
        struct { uint32_t dst, src, rows, cols; float eps; uint32_t src_offset, dst_offset; } layernorm;
        struct { uint32_t dst, src, rows, cols; float eps; uint32_t src_offset, dst_offset; } rmsnorm;
        struct { uint32_t op, dst, src, n_out, reduce_size, src_offset, dst_offset; } reduce;
        struct {
            uint32_t dst, src, n;
            uint32_t src_ne[4], dst_ne[4], src_strides[4], dst_strides[4];
            uint32_t src_offset, dst_offset;
        } repeat;
        struct {
            uint32_t dst, src, rows, cols;
            uint32_t dst_base_offset, dst_offset, dst_row_stride, dst_col_stride;
            uint32_t src_offset, src_row_stride, src_col_stride, patch_stride;
        } slice_assign;
        struct {
            uint32_t dst, src, cos_sin, half_d, seq_len;
            uint32_t src_off, cs_off, dst_off, src_rs, src_cs, cs_cs;
        } rope;
        struct {
            uint32_t dst, q, k, v, mask, has_mask;
            uint32_t d_head, seq_q, seq_kv;
            float scale;
            uint32_t q_off, k_off, v_off, mask_off, dst_off;
            uint32_t q_rs, q_cs, k_rs, k_cs, v_rs, v_cs, mask_rs, mask_cs, dst_rs, dst_cs;
        } attention;
        struct {
            const ZgFusedEwStep* steps;
            size_t n_steps;
            uint32_t n, dst, src, dst_offset, src_offset;
        } fused_elementwise;
        struct { uint32_t buf, offset, n; } allreduce;
        struct { uint32_t dst, src, n, dst_offset, src_offset; } allgather;
        ZgSeqOp seq;
    } u;
} ZgOp;

/* ProgramIO — reference src/backend.zig:252-257.  offset/size in BYTES. */
typedef struct ZgIO {
    uint32_t buf_idx;
    uint32_t offset;
    void* host_ptr;
    uint32_t size;
    uint32_t _pad;
} ZgIO;

/* QuantizedWeightUpload — reference src/backend.zig:260-266.
 * data: i8 [rows*cols] row-major [K=rows, N=cols]; scales: f32, one per
 * `block_size` consecutive FLAT elements (scale index = (k*N+n)/block_size,
 * reference src/quant.zig:525, src/backend/reference.zig:547). */
typedef struct ZgQWeight {
    const int8_t* data;
    size_t n_data;
    const float* scales;
    size_t n_scales;
    size_t rows, cols, block_size;
} ZgQWeight;

/* Extension (direct GGUF->device upload): a descriptor with block_size == ZG_QWEIGHT_RESIDENT
 * refers to a weight already packed in HBM — `data` is the ZgCudaQWeight* that zg_cuda_qweight_upload /
 * zg_cuda_qweight_upload_gguf returned, rows/cols must match it, the other fields are ignored.  The program
 * borrows it (the caller frees it after zg_cuda_free).  Lets a loader stream a model into HBM one tensor at a
 * time instead of holding every expanded i8 copy in host memory until compile (70B: 69.5 GB). */
#define ZG_QWEIGHT_RESIDENT ((size_t)-1)

/* Extension: a program buffer that lives OUTSIDE the program — caller-owned device memory (zg_cuda_malloc) that several
 * programs of one session share: dense weights, per-sequence state.  The program neither zero-fills nor frees it;
 * buffer_sizes[buf_idx] must equal `elems`. */
typedef struct ZgExternBuffer {
    uint32_t buf_idx;
    uint32_t _pad;
    void* device_ptr;   /* 16-byte aligned */
    size_t elems;       /* f32 slots */
} ZgExternBuffer;

/* DeviceProgram — reference src/backend.zig:270-275. buffer_sizes in f32 elements. */
typedef struct ZgProgram {
    const ZgOp* ops;
    size_t n_ops;
    size_t n_buffers;
    const size_t* buffer_sizes;
    const ZgIO* initial_uploads;
    size_t n_uploads;
    const ZgQWeight* qweights;
    size_t n_qweights;
    const ZgExternBuffer* externs;   /* extension; NULL / 0 for the reference's programs */
    size_t n_externs;
} ZgProgram;

/* Subset of RuntimeProfile (reference src/profile.zig:819-842) that a CUDA
 * backend can fill: per-tag device time + counters. */
typedef struct ZgProfile {
    uint64_t time_ns[ZG_OP_COUNT];
    uint64_t backend_op_count;
    uint64_t fallback_op_count;     /* always 0: there is no CPU fallback */
    uint64_t backend_dispatch_count; /* kernels / graph launches issued */
    uint64_t sync_time_ns;
    uint64_t sync_count;
    uint32_t call_count;
    uint32_t _pad;
} ZgProfile;

/* Capabilities to advertise (reference src/backend.zig:14-70). */
typedef struct ZgCapabilities {
    uint32_t compiled_programs, host_visible_program_memory, dense_matmul_f32, dense_matmul_f16;
    uint32_t qmatmul, fused_elementwise, max_fused_elementwise_steps /* 0 = unlimited */;
    uint32_t dynamic_program_refresh, prefill_attention, decode_attention, quantized_kv;
    uint32_t attention_supported, attention_max_seq_kv /* 0 = unlimited */, attention_max_d_head;
} ZgCapabilities;

typedef struct ZgCudaCtx ZgCudaCtx;
typedef struct ZgCudaProgram ZgCudaProgram;

/* ── The six vtable slots + lifecycle ─────────────────────────────────────── */

/* Backend construction (MetalBackend.init analogue, src/backend/metal.zig).
 * NULL when no CUDA device / wrong arch; see zg_cuda_last_error(). */
ZgCudaCtx* zg_cuda_create(int device_ordinal);
void zg_cuda_destroy(ZgCudaCtx* ctx);
void zg_cuda_capabilities(ZgCapabilities* out);

/* VTable.dense_matmul_f32 (src/backend.zig:341): host-pointer GEMM override
 * during graph execution.  Always declines (returns 0) like the fake backend in
 * src/device_inference.zig:750-752: host tensors are not device resident. */
int zg_cuda_dense_matmul_f32(ZgCudaCtx* ctx, float* dst, const float* a, const float* b,
                             const ZgMatMulGeometry* geom);

/* VTable.compile_program (src/backend.zig:343): allocate zero-filled device
 * buffers, apply initial_uploads, copy+repack every qweight into its
 * GPU-resident packed layout, copy the op list.  NULL on any failure. */
ZgCudaProgram* zg_cuda_compile(ZgCudaCtx* ctx, const ZgProgram* program);

/* VTable.refresh_program (src/backend.zig:345): caller's op array after
 * patchSliceAssignOffset / patchAttentionSeqKV (src/device_inference.zig:242-256). */
void zg_cuda_refresh(ZgCudaCtx* ctx, ZgCudaProgram* prog, const ZgOp* ops, size_t n_ops);

/* VTable.execute_program (src/backend.zig:347): upload inputs, run all ops in
 * order, download outputs.  Synchronous: outputs valid on return. */
void zg_cuda_execute(ZgCudaCtx* ctx, ZgCudaProgram* prog, const ZgIO* inputs, size_t n_inputs,
                     const ZgIO* outputs, size_t n_outputs);

/* VTable.free_program (src/backend.zig:349). */
void zg_cuda_free(ZgCudaCtx* ctx, ZgCudaProgram* prog);

/* VTable.get_runtime_profile (src/backend.zig:351). Enabled with
 * zg_cuda_set_profiling(ctx, 1); NULL otherwise. */
const ZgProfile* zg_cuda_profile(ZgCudaCtx* ctx, ZgCudaProgram* prog);
void zg_cuda_set_profiling(ZgCudaCtx* ctx, int enabled);

/* Error convention: NULL / no-op on failure plus this thread-unsafe string. */
const char* zg_cuda_last_error(void);

/* ── Extensions used by tests / bench (not vtable slots) ──────────────────── */

/* Run work on a caller-owned stream (e.g. torch's) instead of the ctx's own. */
void zg_cuda_set_stream(ZgCudaCtx* ctx, void* cuda_stream);
void zg_cuda_sync(ZgCudaCtx* ctx);
/* Kernels launched by this library since process start (claim for gpu_launches). */
uint64_t zg_cuda_launch_count(void);
/* 0: eager launches; 1 (default): capture the op list into a CUDA graph. */
void zg_cuda_set_graph_mode(ZgCudaCtx* ctx, int enabled);
/* Device pointer of program buffer `buf_idx` (for device-resident benches). */
void* zg_cuda_program_buffer(ZgCudaProgram* prog, uint32_t buf_idx);
/* Schedule introspection (tests / benches assert that the fast paths are the ones that run): what == 0: kernels one
 * execution launches (graph nodes); 1: DeviceOps covered by the fused single-token decode kernel (0: general schedule);
 * 2: layers inside that kernel; 3: launches of the streamed single-row matvec kernel (csrc/qgemv_stream.cu) among them;
 * 4: HBM bytes per execution saved by promoted dense operands (zg_cuda_program_promote_dense); 5: waits the tensor-core dense
 * matmul has given up on since process start (0 in a healthy run); 6: LINEAR ops of the program that run on the tensor cores. */
uint64_t zg_cuda_program_stats(const ZgCudaProgram* prog, int what);
/* Run the program's ops with no host<->device copies (inputs already resident);
 * asynchronous on the ctx stream. */
void zg_cuda_execute_device(ZgCudaCtx* ctx, ZgCudaProgram* prog);

/* Packed, GPU-resident quantized weight (the src/quant.zig QuantizedWeight
 * analogue).  Residency format is chosen losslessly at upload:
 *   ZG_QFMT_I8_F32  36 B / 32 weights  (native fromSlice output)
 *   ZG_QFMT_I8_F16  34 B / 32 weights  (every scale is exactly an f16: Q8_0 origin)
 *   ZG_QFMT_I4_F16  18 B / 32 weights  (additionally all q in [-8,7]: Q4_0 origin)
 *   ZG_QFMT_GENERIC block_size != 32 or N % 32 != 0: flat i8 + f32 scales */
enum { ZG_QFMT_AUTO = 0, ZG_QFMT_I8_F32 = 1, ZG_QFMT_I8_F16 = 2, ZG_QFMT_I4_F16 = 3, ZG_QFMT_GENERIC = 4 };
typedef struct ZgCudaQWeight ZgCudaQWeight;

ZgCudaQWeight* zg_cuda_qweight_upload(ZgCudaCtx* ctx, const ZgQWeight* w, int fmt_hint);
/* Direct GGUF block upload (reference src/models/gguf_loader.zig:99-154 done on
 * device): raw = n_blocks * 34 B (ggml_type 8 = Q8_0) or 18 B (2 = Q4_0);
 * rows = dims[0] = K, cols = dims[1] = N, zgml nibble order. */
ZgCudaQWeight* zg_cuda_qweight_upload_gguf(ZgCudaCtx* ctx, const void* raw, size_t raw_bytes,
                                           uint32_t ggml_type, size_t rows, size_t cols);
/* Extension for benchmarks / multi-GPU tests: random-init GGUF blocks generated IN HBM for the slab
 * [k0, k1) x [n0, n1) of a global [rows_full, cols_full] tensor, then imported like zg_cuda_qweight_upload_gguf.
 * Block bytes are a pure function of (seed, tensor_id, global block index): every world size holds slices of the
 * same model, and zgml_b200/host/llama.py::synth_gguf_blocks reproduces them on the host for the CPU oracle. */
ZgCudaQWeight* zg_cuda_qweight_synth_gguf(ZgCudaCtx* ctx, uint64_t seed, uint64_t tensor_id, uint32_t ggml_type,
                                          size_t rows_full, size_t cols_full, size_t k0, size_t k1, size_t n0, size_t n1);
void zg_cuda_qweight_free(ZgCudaCtx* ctx, ZgCudaQWeight* w);
int zg_cuda_qweight_format(const ZgCudaQWeight* w);
size_t zg_cuda_qweight_device_bytes(const ZgCudaQWeight* w);
/* dequantizeTo (src/quant.zig:594-618) from the packed residency: host_dst gets
 * rows*cols f32, bit-exact with the reference.  Returns 0 on success. */
int zg_cuda_qweight_dequantize(ZgCudaCtx* ctx, const ZgCudaQWeight* w, float* host_dst);
/* QuantizedWeight.matmul (src/quant.zig:475-578) with the DeviceOp.qmatmul
 * stride contract, on DEVICE pointers; async on the ctx stream. */
int zg_cuda_qmatmul_device(ZgCudaCtx* ctx, const ZgCudaQWeight* w, const float* d_input,
                           float* d_dst, uint32_t M, uint32_t input_row_stride,
                           uint32_t dst_row_stride);
/* Same through HOST buffers (copies inside): the e2e leg. Synchronous. */
int zg_cuda_qmatmul_host(ZgCudaCtx* ctx, const ZgCudaQWeight* w, const float* h_input,
                         float* h_dst, uint32_t M);

/* QuantizedWeight.fromSlice / fromTensor — reference src/quant.zig:216-264 — on device: quantizes a host f32 [rows=K, cols=N]
 * row-major matrix per flat block of `block_size` (scale = max_abs / 127, q = trunc(clamp(v * 127 / max_abs))) and packs it.
 * h_data_out [rows*cols] / h_scales_out [ceil(rows*cols / block_size)] (either may be NULL) receive the reference's flat
 * form, bit-identical to the CPU result.  NULL on failure. */
ZgCudaQWeight* zg_cuda_qweight_from_f32(ZgCudaCtx* ctx, const float* h_weights, size_t rows, size_t cols, size_t block_size,
                                        int8_t* h_data_out, float* h_scales_out);
/* QuantizedWeight.matmulBias — reference src/quant.zig:581-589: matmul, then dst[m, n] += bias[n] (host buffers). */
int zg_cuda_qmatmul_bias_host(ZgCudaCtx* ctx, const ZgCudaQWeight* w, const float* h_input, const float* h_bias,
                              float* h_dst, uint32_t M);

/* W8A8 decode path (what `session.quantize()` models run per linear on the reference's aarch64 builds).  All three are
 * integer / IEEE-exact work and bit-identical to the reference.
 * prepareTransposed — reference src/quant.zig:274-317 (twin src/backend/reference.zig:26-70): dequantize [K, N], re-quantize
 * into [N, K] int8 with K-aligned blocks + [N, ceil(K / block_size)] f32 scales; both stay resident with the weight.
 * h_t_data / h_t_scales (either may be NULL) receive copies.  Idempotent.  Returns 0 on success. */
int zg_cuda_qweight_prepare_transposed(ZgCudaCtx* ctx, ZgCudaQWeight* w, int8_t* h_t_data, float* h_t_scales);
/* quantizeInput — reference src/quant.zig:320-341: per K-block scale = max_abs / 127 (1 if zero),
 * q = trunc(clamp(v * (127 / max_abs), +-127)).  Host buffers: h_q [K], h_scales [ceil(K / block_size)].
 * Limits as the reference's stack buffers (src/quant.zig:452-453): K <= 16384, <= 512 blocks. */
int zg_cuda_quantize_input_host(ZgCudaCtx* ctx, const float* h_input, size_t K, size_t block_size, int8_t* h_q, float* h_scales);
/* gemv — reference src/quant.zig:443-459 = quantizeInput + gemvRange (:358-440) over all N outputs, M = 1:
 * dst[n] = sum over K-blocks ascending of f32(int32 dot) * (s_x[b] * s_w[n, b]).  Needs prepare_transposed.
 * _device: device pointers, async on the ctx stream; _host: host buffers, synchronous. */
int zg_cuda_gemv_w8a8_device(ZgCudaCtx* ctx, const ZgCudaQWeight* w, const float* d_input, float* d_dst);
int zg_cuda_gemv_w8a8_host(ZgCudaCtx* ctx, const ZgCudaQWeight* w, const float* h_input, float* h_dst);

/* Quantized KV cache + attention over it — reference src/quant.zig:633-1091, callers
 * src/llama_inference.zig:330-377.  Column-major Q8 cache: column c = d_head int8 + d_head / block_size f32 scales; one
 * column per kv position inside a head's slab.  d_head <= 512 and d_head % block_size == 0 as in the reference; this
 * implementation additionally needs d_head % 4 == 0 and block_size % 4 == 0. */
typedef struct ZgCudaKVCache ZgCudaKVCache;
/* QuantizedKVCache.init / deinit / clear — src/quant.zig:658-686 (zero-filled). NULL on failure. */
ZgCudaKVCache* zg_cuda_kvcache_create(ZgCudaCtx* ctx, size_t d_head, size_t n_cols, size_t block_size);
void zg_cuda_kvcache_free(ZgCudaCtx* ctx, ZgCudaKVCache* cache);
int zg_cuda_kvcache_clear(ZgCudaCtx* ctx, ZgCudaKVCache* cache);
/* storeColumn — src/quant.zig:689-701 — for n_write consecutive columns from src [n_write][d_head] (the slice_assign
 * routing of src/llama_inference.zig:336-348): quantizeInput per column, bit-identical data and scales.
 * _device: device pointer, async on the ctx stream; _host: host buffer, synchronous. */
int zg_cuda_kvcache_store_device(ZgCudaCtx* ctx, ZgCudaKVCache* cache, size_t col_start, size_t n_write, const float* d_src);
int zg_cuda_kvcache_store_host(ZgCudaCtx* ctx, ZgCudaKVCache* cache, size_t col_start, size_t n_write, const float* h_src);
/* whole cache to the host: h_q [d_head * n_cols], h_scales [d_head / block_size * n_cols] (either may be NULL) */
int zg_cuda_kvcache_download(ZgCudaCtx* ctx, const ZgCudaKVCache* cache, int8_t* h_q, float* h_scales);
/* attentionQuantized — src/quant.zig:924-1091, same argument meaning: q / dst column-major [d_head, seq_q] with column
 * strides, kv columns [col_start, col_start + seq_kv) of each cache, optional additive mask [seq_kv, seq_q or 1] with
 * (row, column) strides (column stride 0 broadcasts one column; non-finite entries skip the position; a fully masked
 * query column yields zeros).  int8_query != 0: the aarch64 branch (query quantized per block, int8 x int8 scores);
 * 0: the portable branch (f32 query x int8 keys).  Scores are bit-identical to the reference's; the softmax groups
 * positions differently, so outputs agree to float rounding. */
int zg_cuda_attention_quantized_device(ZgCudaCtx* ctx, float* d_dst, size_t dst_col_stride, const float* d_q, size_t q_col_stride,
                                       size_t d_head, size_t seq_q, const ZgCudaKVCache* k_cache, size_t k_col_start,
                                       const ZgCudaKVCache* v_cache, size_t v_col_start, size_t seq_kv, const float* d_mask,
                                       size_t mask_row_stride, size_t mask_col_stride, float scale, int int8_query);
int zg_cuda_attention_quantized_host(ZgCudaCtx* ctx, float* h_dst, size_t dst_col_stride, const float* h_q, size_t q_col_stride,
                                     size_t d_head, size_t seq_q, const ZgCudaKVCache* k_cache, size_t k_col_start,
                                     const ZgCudaKVCache* v_cache, size_t v_col_start, size_t seq_kv, const float* h_mask,
                                     size_t mask_row_stride, size_t mask_col_stride, float scale, int int8_query);

/* LlamaInferenceSession.quantizeKV for a compiled program — src/llama_inference.zig:648-679 (plan side :277-328): from now on
 * every patched slice_assign into a buffer that attention ops read as K or V stores quantized columns (storeColumn) into a
 * Q8 cache standing in for that buffer, and those attention ops run attentionQuantized over the caches (the routing of
 * src/llama_inference.zig:336-377).  The caches start zeroed, like the reference's; call it right after compile.
 * int8_query != 0: the aarch64 branch of attentionQuantized (query quantized per block), 0: the portable f32-query branch.
 * Returns 0 on success; -1 (program unchanged) when the program's cache accesses are not whole d_head columns. */
int zg_cuda_program_quantize_kv(ZgCudaCtx* ctx, ZgCudaProgram* prog, size_t block_size, int int8_query);

/* Format hint for dense matmul operands (precedent: the WGPU backend's f16 promotion of matmul B buffers that
 * have initial uploads, src/backend/wgpu.zig:1068-1106).  Every matmul op of the program with M == 1 and a k-contiguous B
 * operand that no op writes (the tied LM head x @ token_embed^T, src/models/llama.zig:162-165) gets a 16-bit copy of that operand;
 * the op then streams the copy (half the bytes), bounds each output's error by ||x|| * ||w - round16(w)|| and recomputes every
 * column that could still be the maximum from the f32 original, with the exact kernel's arithmetic.  The argmax — and the
 * winning logits bit for bit — equal the unpromoted program's; the other outputs carry the 16-bit weight rounding.
 * An execute() input that overwrites a promoted operand refreshes its copy.  Returns the number of ops promoted, -1 on error. */
#define ZG_DENSE_BF16 1   /* f32's range, 8 significant bits: other logits within ~2e-3 of the output scale */
#define ZG_DENSE_F16 2    /* the WGPU backend's choice, 11 significant bits: other logits within ~2e-4; |w| > 65504 falls back to the exact row */
int zg_cuda_program_promote_dense(ZgCudaCtx* ctx, ZgCudaProgram* prog, int format);

/* Multi-GPU (one process per GPU): a 128-byte NCCL unique id made on rank 0, distributed by the host
 * (torch.distributed / MPI / file), then one communicator per context.  Returns 0 on success. */
int zg_cuda_comm_unique_id(void* id128);
int zg_cuda_comm_init(ZgCudaCtx* ctx, const void* id128, int rank, int world);
void zg_cuda_comm_destroy(ZgCudaCtx* ctx);
/* 0 = no communicator, 1 = NCCL only, 2 = small all-reduces over NVLink peer memory (cudaIpc) + NCCL for the rest. */
int zg_cuda_comm_mode(const ZgCudaCtx* ctx);

/* Debug timeline of a program's kernels (off by default): records of 3 x u64 {kind << 56 | t_entry, t_after_wait, t_exit},
 * %globaltimer ns stamped by block 0 of each kernel; kinds: 1 elementwise, 2 fused_elementwise, 3 rmsnorm, 4 repeat,
 * 5 slice_assign, 6 rope, 7 attention, 8 chain, 9 dense matmul, 10 quantized matvec. */
int zg_cuda_trace(ZgCudaCtx* ctx, int enable);
size_t zg_cuda_trace_read(ZgCudaCtx* ctx, unsigned long long* host, size_t max_records);

/* f32 slots the scratch operand of a sequence-model op must have (MOE_FFN buf[4]: per-pair activations, or the sorted
 * rows, per-expert tiles and partial products of the grouped tensor-core form); 0 for ops without one. */
size_t zg_cuda_seq_scratch_elems(const ZgOp* op);
/* f32 slots per state slot of a sequence-model op that lays out its own state (SSM_SCAN, from H, N and P); 0 otherwise. */
size_t zg_cuda_seq_state_elems(const ZgOp* op);

void* zg_cuda_malloc(ZgCudaCtx* ctx, size_t bytes);
void zg_cuda_free_device(ZgCudaCtx* ctx, void* p);
int zg_cuda_memcpy_h2d(ZgCudaCtx* ctx, void* d, const void* h, size_t bytes);
int zg_cuda_memcpy_d2h(ZgCudaCtx* ctx, void* h, const void* d, size_t bytes);
int zg_cuda_memset(ZgCudaCtx* ctx, void* d, int value, size_t bytes);

#ifdef __cplusplus
}
#endif
#endif /* ZGML_CUDA_H */
