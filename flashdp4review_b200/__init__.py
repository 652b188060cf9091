"""B200-native DP-SGD backward path behind the FlashDP Python API.

`wrap_with_flashdp_layers`, `DPLinear`, `DPConv1D`, `DPLayerNorm` mirror the reference package
(flashdp/__init__.py:1-8); the kernels live in libfdp_b200.so (sm_100a, C ABI in include/fdp_b200.h).
"""
from .layers.linear import DPLinear
from .layers.layernorm import DPLayerNorm
from .layers.transformers_conv1d import DPConv1D
from .api.wrap_model import wrap_with_flashdp_layers, dp_supported_modules
from .runtime import (manual_seed, set_data_parallel, set_input_grad_impl, set_accumulation, accumulate,
                      noise_state, set_noise_state, check_device_status, clear_device_status, sm_reservation,
                      set_fp32_mode, fp32_mode, use_device_noise_step, advance_noise_step)

__all__ = ["DPLinear", "DPLayerNorm", "DPConv1D", "wrap_with_flashdp_layers", "dp_supported_modules",
           "manual_seed", "set_data_parallel", "set_input_grad_impl", "set_accumulation", "accumulate",
           "noise_state", "set_noise_state", "check_device_status", "clear_device_status", "sm_reservation", "set_fp32_mode", "fp32_mode",
           "use_device_noise_step", "advance_noise_step"]
