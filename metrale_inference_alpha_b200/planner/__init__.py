from .roofline import DevicePeaks, LayerOp, decode_step_ops, estimate, load_peaks  # noqa: F401
