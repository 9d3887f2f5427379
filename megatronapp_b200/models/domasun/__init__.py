from .config import DomasunConfig  # noqa: F401
from .loader import load_model_dir  # noqa: F401
from .model import DomasunModel  # noqa: F401
