"""Layer-level mirrors of xax/nn (FP8 linear)."""
