"""Checkpoint / model file formats: RusTorch binary container, safetensors, PyTorch state dicts, GGUF."""
from . import gguf, rustorch_bin, safetensors  # noqa: F401
from .safetensors import (detect_format, load_huggingface, load_json_state_dict, load_pth, load_safetensors,
                          save_huggingface, save_json_state_dict, save_pth, save_safetensors, save_torch_state_dict)
