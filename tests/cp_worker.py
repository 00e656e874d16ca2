"""torchrun worker: ring attention on the flash kernels over NCCL against full attention in fp32 (one GPU per rank)."""
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from rustorch_b200.distributed.context_parallel import gather_sequence, ring_attention, shard_sequence  # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dist.init_process_group("nccl")
    dev = torch.device("cuda")
    res = {}
    for D, H, Hkv in ((64, 4, 4), (128, 4, 2)):
        g = torch.Generator(device=dev).manual_seed(7)
        B, T = 2, 256 * world
        q = (torch.randn(B, T, H, D, device=dev, generator=g) * 0.5).bfloat16()
        k = (torch.randn(B, T, Hkv, D, device=dev, generator=g) * 0.5).bfloat16()
        v = (torch.randn(B, T, Hkv, D, device=dev, generator=g) * 0.5).bfloat16()
        go = (torch.randn(B, T, H, D, device=dev, generator=g) * 0.5).bfloat16()
        for causal in (False, True):
            qf, kf, vf = (t.float().requires_grad_(True) for t in (q, k, v))
            s = (qf.transpose(1, 2) @ kf.repeat_interleave(H // Hkv, 2).transpose(1, 2).transpose(-1, -2)) / D ** 0.5
            if causal:
                s = s.masked_fill(torch.ones(T, T, dtype=torch.bool, device=dev).triu(1), float("-inf"))
            ref = (torch.softmax(s, -1) @ vf.repeat_interleave(H // Hkv, 2).transpose(1, 2)).transpose(1, 2)
            ref.backward(go.float())
            ql, kl, vl = (shard_sequence(t).requires_grad_(True) for t in (q, k, v))
            att = ring_attention(ql, kl, vl, causal=causal)
            att.backward(shard_sequence(go))
            tag = f"d{D}_{'causal' if causal else 'full'}"

            def rel(a, b):
                return float((a.float() - b).abs().max() / b.abs().max())
            res[f"{tag}_fwd"] = rel(gather_sequence(att.detach()), ref.detach())
            res[f"{tag}_dq"] = rel(gather_sequence(ql.grad), qf.grad)
            res[f"{tag}_dk"] = rel(gather_sequence(kl.grad), kf.grad)
            res[f"{tag}_dv"] = rel(gather_sequence(vl.grad), vf.grad)
    from rustorch_b200 import _native
    _native.check_status()
    res["launches"] = _native.launch_count()
    with open(os.path.join(os.environ["CP_RESULT_DIR"], f"rank{rank}.json"), "w") as f:
        json.dump(res, f)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
