from .wrap_model import wrap_with_flashdp_layers, dp_supported_modules  # noqa: F401
