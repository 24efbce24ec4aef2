from .flow_match import FlowMatchScheduler  # noqa: F401
from .registry import ENCODERS, MODELS, build_model, encoder_for_model, get_encoder  # noqa: F401
from .wan import WAN_PRESETS, WanConfig, WanModel, wan_config  # noqa: F401
from . import parallel_wan  # noqa: F401  (registers ParallelWanModel)
from .hunyuan import HUNYUAN_PRESETS, HunyuanConfig, HunyuanVideoModel, ParallelHunyuanVideoModel, hunyuan_config  # noqa: F401,E402
from . import encoders  # noqa: F401,E402  (registers wan_encoder)
