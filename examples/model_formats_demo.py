"""Round trips through the supported model formats: safetensors, PyTorch state dict, RusTorch binary container, GGUF."""
import _path  # noqa: F401
import os
import tempfile

import torch

from rustorch_b200 import formats, nn
from rustorch_b200.formats import gguf, rustorch_bin

torch.manual_seed(0)
model = nn.Sequential(nn.Linear(64, 32), nn.ReLU(), nn.Linear(32, 4))
sd = {k: v.detach() for k, v in model.state_dict().items()}
with tempfile.TemporaryDirectory() as d:
    st = os.path.join(d, "m.safetensors")
    formats.save_safetensors(sd, st)
    back = formats.load_safetensors(st)
    print("safetensors:", formats.detect_format(st), all(torch.equal(sd[k], back[k]) for k in sd))

    pth = os.path.join(d, "m.pth")
    formats.save_pth(sd, pth)
    print("pth:", all(torch.equal(sd[k], v) for k, v in formats.load_pth(pth).items()))

    rt = os.path.join(d, "m.rustorch")
    rustorch_bin.save_module(model, rt, model_type="mlp")
    clone = nn.Sequential(nn.Linear(64, 32), nn.ReLU(), nn.Linear(32, 4))
    meta = rustorch_bin.load_module(clone, rt)
    print("rustorch binary:", rustorch_bin.is_rustorch_file(rt), torch.equal(clone[0].weight, model[0].weight), sorted(meta)[:3])

    gg = os.path.join(d, "m.gguf")
    w = torch.randn(8, 64)
    gguf.write_gguf(gg, {"general.architecture": "llama", "llama.block_count": 1},
                    {"w_f32": (w, gguf.GGMLType.F32), "w_q4": (w, gguf.GGMLType.Q4_0), "w_q8": (w, gguf.GGMLType.Q8_0)})
    with gguf.GGUFFile(gg) as f:
        print("gguf:", f.architecture(), "f32 exact:", torch.equal(f.load_tensor("w_f32"), w),
              "q8 max err: %.4f" % float((f.load_tensor("w_q8") - w).abs().max()),
              "q4 max err: %.4f" % float((f.load_tensor("w_q4") - w).abs().max()))
