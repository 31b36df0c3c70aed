"""Vision input path: image decoding and preprocessing (``preprocess``), the ViT tower with its patch
merger (``encoder``) and the multimodal position index (``mrope``). Reference: the vision stack of
``crates/model-layers`` and ``kernels/gb10/qwen3-vl-30b-a3b/nvfp4/vision_encoder.cu``."""
from .encoder import VisionConfig, VisionEncoder  # noqa: F401
from .preprocess import ImagePreprocessor, smart_resize  # noqa: F401
from .mrope import mrope_positions  # noqa: F401
