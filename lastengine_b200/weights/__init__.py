from .loader import check_names, load_model_dir, load_random  # noqa: F401
from .random_init import write_model_dir  # noqa: F401
from .safetensors_io import SafetensorsFile, WeightsError, open_checkpoint, save_file  # noqa: F401
