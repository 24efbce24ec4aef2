from .clip_vit import VisionTransformer, WanImageEncoder  # noqa: F401
from .umt5 import UMT5Encoder, encode_prompt  # noqa: F401
from .wan_encoder import WanVideoEncoder  # noqa: F401
from .wan_vae import WanVideoVAE  # noqa: F401
