"""Checkpoint / model file formats: RusTorch binary container, safetensors, PyTorch state dicts, GGUF, MLX."""
from . import gguf, mlx, rustorch_bin, safetensors  # noqa: F401
from .mlx import MLXLoader, load_mlx, save_mlx  # noqa: F401
from .safetensors import (detect_format, load_huggingface, load_json_state_dict, load_pth, load_safetensors,
                          save_huggingface, save_json_state_dict, save_pth, save_safetensors, save_torch_state_dict)
