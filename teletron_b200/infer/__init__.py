from .wan_pipeline import WanVideoPipeline  # noqa: F401
from .hunyuan_pipeline import HunyuanVideoPipeline  # noqa: F401
