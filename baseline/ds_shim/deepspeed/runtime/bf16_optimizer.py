class BF16_Optimizer:
    """Marker base class: the stand-in engine's optimizer wrapper derives from it in bf16 mode."""
