/* The linear dispatch of one DiT block, in C above the operator interface.
 *
 * The reference's run_block() (src/denoise/dit.c:2286-2537) decides per projection which operator
 * family runs it -- the int8 (W8A8) entry points, or h3_gpu_linear_bf16 on a bf16 tensor or a
 * quantised descriptor -- from flags fixed at load time (src/denoise/dit.c:1956-1990) and a few
 * H3_DISABLE_* switches, and it carries one piece of state from operator to operator: whether the
 * int8 activation buffer already holds the quantised input of the next linear
 * (attention_input_quantized / next_attention_input_quantized, :2289-2292, 2513).  This file is that
 * logic for the four projections and the element operators between them; attention itself sits
 * between the two calls and stays with the caller.
 *
 * Plain C on purpose: it uses nothing but the functions include/h3q8.h declares, the way dit.c does.
 */
#include <stdlib.h>
#include <string.h>

#include "h3q8.h"

/* ---------------------------------------------------------------- which matrices are quantised */
/* src/weights/quant.c:22-30: only blocks.<index>.{attn.qkv_proj, attn.out_proj, mlp.fc1, mlp.fc2}.weight */
int h3_quant_projection(const char *name, int requested) {
    static const char *const projections[] = {"attn.qkv_proj.weight", "attn.out_proj.weight", "mlp.fc1.weight", "mlp.fc2.weight"};
    static const char prefix[] = "blocks.";
    if (!name || strncmp(name, prefix, sizeof prefix - 1)) return 0;
    const char *cursor = name + sizeof prefix - 1;
    size_t digits = strspn(cursor, "0123456789");
    if (!digits || cursor[digits] != '.') return 0;
    cursor += digits + 1;
    for (size_t i = 0; i < sizeof projections / sizeof projections[0]; i++)
        if (!strcmp(cursor, projections[i])) return requested;
    return 0;
}
/* src/weights/quant.c:37-40: with the adaptive cache block 0 keeps its bf16 weights */
int h3_quant_projection_policy(const char *name, int requested, int adaptive_cache) {
    if (adaptive_cache && name && !strncmp(name, "blocks.0.", 9)) return 0;
    return h3_quant_projection(name, requested);
}

/* ---------------------------------------------------------------- policy */
static int disabled(const char *variable) { return getenv(variable) != NULL; }

int h3q8_dit_linear_policy_resolve(const h3_gpu *gpu, uint32_t rows, int streaming, h3q8_dit_linear_policy *policy) {
    if (!policy) return 0;
    memset(policy, 0, sizeof *policy);
    /* src/denoise/dit.c:1956-1968: the int8 family needs the backend's int8 operators, resident weights and, for the
     * attention-side projections, at least one 128-row tile */
    const int available = !streaming && h3_gpu_has_int8_mlp(gpu);
    policy->int8_mlp = available && !disabled("H3_DISABLE_INT8_MLP");
    policy->int8_qkv = available && rows >= 128 && !disabled("H3_DISABLE_INT8_QKV");
    policy->int8_attention_out = available && rows >= 128 && !disabled("H3_DISABLE_INT8_ATTENTION_OUT");
    policy->head_major_attention_out = policy->int8_attention_out && !disabled("H3_DISABLE_HEAD_MAJOR_ATTENTION_OUTPUT");
    policy->fuse_int8_mlp_input = policy->int8_mlp && !disabled("H3_DISABLE_FUSED_INT8_MLP_INPUT") && !disabled("H3_INT8_MLP_STAGE");
    policy->fuse_int8_qkv_input = policy->int8_qkv && !disabled("H3_DISABLE_FUSED_INT8_QKV_INPUT");
    policy->int8_row_fc2 = 0;
    return 1;
}

/* ---------------------------------------------------------------- first half: up to the attention inputs */
int h3q8_dit_block_attention_input(h3_gpu *gpu, const h3q8_dit_linear_policy *policy, const h3q8_dit_shape *shape,
                                   const h3q8_dit_block_weights *weights, const h3q8_dit_block_buffers *buffers,
                                   const h3_gpu_tensor *modulation, const h3_gpu_tensor *row_map, const h3_gpu_tensor *rope_cos,
                                   const h3_gpu_tensor *rope_sin, int attention_adaln_ready, int attention_input_quantized) {
    if (!gpu || !policy || !shape || !weights || !buffers) return 0;
    const uint32_t rows = shape->rows, hidden = shape->hidden;
    /* slots 0 / 1: shift and scale of the attention AdaLN (src/denoise/dit.c:2346-2349) */
    if (!attention_adaln_ready &&
        !h3_gpu_adaln_bf16(gpu, buffers->mod_attention, buffers->hidden, weights->norm1, modulation, row_map, rows, hidden, shape->slots,
                           0, 1, shape->epsilon))
        return 0;
    if (policy->int8_qkv && weights->qkv_int8)   /* :2351-2362; a quantised input is only there when the previous tail left one */
        return h3_gpu_grouped_qkv_linear_rope_int8(gpu, buffers->query, buffers->key, buffers->value, buffers->int8_activation,
                                                   buffers->int8_activation_scales, buffers->mod_attention, weights->qkv_int8,
                                                   weights->qkv_scales, weights->q_norm, weights->k_norm, rope_cos, rope_sin, rows, hidden,
                                                   shape->heads, shape->head_dim, shape->rope_half, shape->epsilon,
                                                   attention_adaln_ready && attention_input_quantized, 0, 0, 0);
    /* :2375-2380: bf16 weight or quantised descriptor behind the same call */
    return h3_gpu_grouped_qkv_linear_rope_bf16(gpu, buffers->query, buffers->key, buffers->value, buffers->qkv, buffers->mod_attention,
                                               weights->qkv, weights->q_norm, weights->k_norm, rope_cos, rope_sin, rows, hidden,
                                               shape->heads, shape->head_dim, shape->rope_half, shape->epsilon);
}

/* ---------------------------------------------------------------- second half: from the attention output to the block output */
int h3q8_dit_block_after_attention(h3_gpu *gpu, const h3q8_dit_linear_policy *policy, const h3q8_dit_shape *shape,
                                   const h3q8_dit_block_weights *weights, const h3_gpu_tensor *next_norm1,
                                   const h3q8_dit_block_buffers *buffers, const h3_gpu_tensor *modulation,
                                   const h3_gpu_tensor *next_modulation, const h3_gpu_tensor *row_map, int fuse_next_attention,
                                   int *next_attention_adaln_ready, int *next_attention_input_quantized) {
    if (!gpu || !policy || !shape || !weights || !buffers) return 0;
    const uint32_t rows = shape->rows, hidden = shape->hidden, inner = shape->heads * shape->head_dim, ffn = shape->ffn;
    const uint32_t padded_rows = (rows + 127u) & ~127u;
    if (next_attention_adaln_ready) *next_attention_adaln_ready = 0;
    if (next_attention_input_quantized) *next_attention_input_quantized = 0;

    /* attention output projection (:2409-2427): head-major int8, row-major int8, or the bf16 / descriptor call */
    const int int8_out = policy->int8_attention_out && weights->out_int8;
    if (int8_out && policy->head_major_attention_out) {
        if (!h3_gpu_linear_int8_head_major_bf16(gpu, buffers->attention_output, buffers->int8_activation, buffers->int8_activation_scales,
                                                buffers->attention_heads, weights->out_int8, weights->out_scales, rows, shape->heads,
                                                shape->head_dim, hidden)) return 0;
    } else if (int8_out) {
        if (!h3_gpu_linear_int8_bf16(gpu, buffers->attention_output, buffers->int8_activation, buffers->int8_activation_scales,
                                     buffers->attention_heads, weights->out_int8, weights->out_scales, rows, inner, hidden, 0)) return 0;
    } else if (!h3_gpu_linear_bf16(gpu, buffers->attention_output, buffers->attention_heads, weights->out, NULL, rows, inner, hidden)) return 0;

    /* gate (slot 2) into the residual stream, MLP AdaLN (slots 3 / 4), and -- when the MLP is int8 -- its quantiser in the
     * same pass (:2433-2458) */
    const int int8_mlp = policy->int8_mlp && weights->fc1_int8 && weights->fc2_int8;
    const int mlp_input_quantized = int8_mlp && policy->fuse_int8_mlp_input;
    if (mlp_input_quantized) {
        if (!h3_gpu_gate_adaln_quantize_int8(gpu, buffers->hidden, buffers->int8_activation, buffers->int8_activation_scales,
                                             buffers->hidden, buffers->attention_output, weights->norm2, modulation, modulation, row_map,
                                             rows, padded_rows, hidden, shape->slots, 2, 3, 4, shape->epsilon)) return 0;
    } else if (!h3_gpu_gate_adaln_bf16(gpu, buffers->hidden, buffers->mod_mlp, buffers->hidden, buffers->attention_output, weights->norm2,
                                       modulation, modulation, row_map, rows, hidden, shape->slots, 2, 3, 4, shape->epsilon)) return 0;

    /* MLP (:2466-2495): fc1 + SwiGLU, re-quantisation, fc2 on the int8 family, else the bf16 / descriptor MLP */
    if (int8_mlp) {
        if (!h3_gpu_mlp_int8_bf16(gpu, buffers->mlp_output, buffers->activated, buffers->int8_activation, buffers->int8_activation_scales,
                                  buffers->mod_mlp, weights->fc1_int8, weights->fc1_scales, weights->fc2_int8, weights->fc2_scales,
                                  weights->fc1, weights->fc2, rows, hidden, ffn, hidden, 0, 0, policy->int8_row_fc2, mlp_input_quantized)) return 0;
    } else if (!h3_gpu_mlp_bf16(gpu, buffers->mlp_output, buffers->mod_mlp, weights->fc1, weights->fc2, rows, hidden, ffn, hidden)) return 0;

    /* MLP gate (slot 5); fused with the NEXT block's attention AdaLN (its slots 0 / 1) and, when that block's QKV is
     * int8, with its quantiser -- which is what the caller passes back in as attention_input_quantized (:2497-2526) */
    if (!fuse_next_attention)
        return h3_gpu_gate_bf16(gpu, buffers->hidden, buffers->hidden, buffers->mlp_output, modulation, row_map, rows, hidden, shape->slots, 5);
    if (!next_norm1 || !next_modulation) return 0;
    if (policy->int8_qkv && policy->fuse_int8_qkv_input) {
        if (!h3_gpu_gate_adaln_quantize_int8(gpu, buffers->hidden, buffers->int8_activation, buffers->int8_activation_scales,
                                             buffers->hidden, buffers->mlp_output, next_norm1, modulation, next_modulation, row_map, rows,
                                             padded_rows, hidden, shape->slots, 5, 0, 1, shape->epsilon)) return 0;
        if (next_attention_input_quantized) *next_attention_input_quantized = 1;
    } else if (!h3_gpu_gate_adaln_bf16(gpu, buffers->hidden, buffers->mod_attention, buffers->hidden, buffers->mlp_output, next_norm1,
                                       modulation, next_modulation, row_map, rows, hidden, shape->slots, 5, 0, 1, shape->epsilon)) return 0;
    if (next_attention_adaln_ready) *next_attention_adaln_ready = 1;
    return 1;
}
