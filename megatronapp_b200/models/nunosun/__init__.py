from .config import NunosunConfig, NunosunLayerConfig  # noqa: F401
from .loader import load_model_dir, load_nunosun_weights  # noqa: F401
from .model import NunosunModel  # noqa: F401
