"""Vision tower: the ViT encoder, its fp32 oracle, the embedding cache and the slice-to-rank job split."""
from .encoder import VisionConfig, VisionEncoder, synth_vision_weights, vision_reference, slice_positions  # noqa: F401
from .cache import VisionCache, assign_slices, media_key  # noqa: F401
from .frontend import VisionFrontend  # noqa: F401
