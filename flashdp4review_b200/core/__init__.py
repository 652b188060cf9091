from .ops import (  # noqa: F401
    linear_weight_flashdp, conv1d_weight_flashdp, linear_bias_grad_clip, bmtm_clip, bmm_clip, mm_clip,
    layernorm_fwd_fused, layernorm_dw_clip, layernorm_db_clip, layernorm_bwd_clip_fused, layernorm_dwdb_fused,
    mm_fused,
    dp_linear_weight_grad, dp_bias_grad, dp_layernorm_backward, linear_input_grad, linear_forward,
    RuntimeAutoTuner, NoiseSpec, noise_std,
)
