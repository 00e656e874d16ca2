"""Per-rank sharded checkpoints: cut, merge, reshard to another world size, asynchronous save."""
import os

import torch

from rustorch_b200 import training
from rustorch_b200.models.llama import LlamaModel, LlamaTrainConfig
from rustorch_b200.training import sharded


def _llama_state():
    torch.manual_seed(0)
    cfg = LlamaTrainConfig.tiny(n_layer=2, n_embd=64, n_head=4, n_head_kv=4, n_ff=128, vocab_size=64)
    m = LlamaModel(cfg, device="cpu", dtype=torch.float32)
    for p in m.parameters():
        p.data.normal_()
    return m, {k: v.detach().clone() for k, v in m.state_dict().items()}


def test_shard_merge_roundtrip_and_reshard(tmp_path):
    model, full = _llama_state()
    spec = sharded.infer_spec(model)
    assert spec["blocks.0.wqkv"].segments == [64, 64, 64] and spec["blocks.1.w_down"].dim == 1
    d = str(tmp_path / "ckpt")
    world = 4
    for r in range(world):
        local = {k: sharded.shard_tensor(v, spec.get(k), r, world) for k, v in full.items()}
        assert local["blocks.0.wqkv"].shape == (48, 64) and local["blocks.0.w_down"].shape == (64, 32)
        sharded.save_sharded(local, d, r, world, spec)
    merged = sharded.merge_sharded(d)
    assert set(merged) == set(full) and all(torch.equal(merged[k], full[k]) for k in full)
    # the q | k | v parts are cut one by one: rank 1 of 4 holds rows 16..31 of q, of k and of v
    r1 = sharded.load_sharded(d, 1, 4)["blocks.0.wqkv"]
    assert torch.equal(r1[:16], full["blocks.0.wqkv"][16:32]) and torch.equal(r1[16:32], full["blocks.0.wqkv"][64 + 16:64 + 32])
    # reshard to two ranks
    two = [sharded.load_sharded(d, r, 2) for r in range(2)]
    again = {k: sharded.merge_tensors([t[k] for t in two], spec.get(k), k) for k in full}
    assert all(torch.equal(again[k], full[k]) for k in full)
    assert sharded.main(["merge", d, str(tmp_path / "merged.safetensors")]) == 0
    from rustorch_b200.formats import load_safetensors
    back = load_safetensors(str(tmp_path / "merged.safetensors"))
    assert all(torch.equal(back[k], full[k]) for k in full)


def test_replicated_mismatch_is_reported(tmp_path):
    a, b = {"w": torch.ones(4)}, {"w": torch.zeros(4)}
    d = str(tmp_path / "bad")
    sharded.save_sharded(a, d, 0, 2, {})
    sharded.save_sharded(b, d, 1, 2, {})
    try:
        sharded.merge_sharded(d)
    except ValueError as e:
        assert "differs" in str(e)
    else:
        raise AssertionError("mismatch between replicated tensors not detected")


def test_column_row_parallel_specs():
    from rustorch_b200.distributed.model_parallel import ColumnParallelLinear, RowParallelLinear, TensorParallel
    tp = TensorParallel(2, 0, -1, None)
    net = torch.nn.Sequential(ColumnParallelLinear(8, 16, tp), RowParallelLinear(16, 8, tp))
    spec = sharded.infer_spec(net)
    assert spec["0.weight"].dim == 0 and spec["0.bias"].dim == 0 and spec["1.weight"].dim == 1 and "1.bias" not in spec


def test_async_checkpointer(tmp_path):
    ck = training.AsyncCheckpointer()
    state = {"a": torch.randn(128, 64), "b": torch.arange(10)}
    p1, p2 = str(tmp_path / "s1.safetensors"), str(tmp_path / "s2.safetensors")
    ck.save(state, p1)
    state["a"].add_(1.0)                        # the first save must have captured the old values
    ck.save(state, p2)
    ck.wait()
    from rustorch_b200.formats import load_safetensors
    one, two = load_safetensors(p1), load_safetensors(p2)
    assert torch.allclose(one["a"] + 1.0, two["a"]) and torch.equal(two["b"], state["b"])
    assert ck.saved == [p1, p2] and not os.path.exists(p1 + ".tmp")
