"""CUDA entry of masked attention (temporary dense path until the kernel lands)."""

from speculators_b200.ops.attention import masked_attention_reference


def masked_attention_cuda(q, k_ctx, v_ctx, spec, k_ext=None, v_ext=None, scale=None):
    return masked_attention_reference(q, k_ctx, v_ctx, spec, k_ext, v_ext, scale)
