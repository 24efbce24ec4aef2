from .registry import DATASETS, build_dataset  # noqa: F401
from .fake import FakeDataset, SyntheticHunyuanDataset, SyntheticLatentDataset, latent_grid  # noqa: F401
from .samplers import (PretrainingRandomSampler, PretrainingSampler, RandomSeedDataset,  # noqa: F401
                       build_data_loader)
from . import synthetic_encoder  # noqa: F401,E402  (registers synthetic_wan_encoder)
from .video_folder import VideoFolderDataset  # noqa: F401,E402
