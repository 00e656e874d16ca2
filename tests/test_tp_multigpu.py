"""Fused all-gather->GEMM and GEMM->reduce-scatter kernels on >= 2 GPUs against the unsharded model."""
import json
import os
import socket
import subprocess
import sys
import tempfile

import pytest
import torch

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_tp_fused_kernels_match_unsharded_model():
    nproc = min(torch.cuda.device_count(), 4)
    if nproc < 2:
        pytest.skip("needs at least 2 GPUs")
    out_dir = tempfile.mkdtemp(prefix="tp_res_")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", TP_RESULT_DIR=out_dir)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}", "--master-addr", "127.0.0.1",
           "--master-port", str(_free_port()), os.path.join(ROOT, "tests", "tp_worker.py")]
    p = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    assert p.returncode == 0, p.stdout[-3000:] + p.stderr[-3000:]
    for r in range(nproc):
        res = json.load(open(os.path.join(out_dir, f"rank{r}.json")))
        assert res["p2p_coll_rel"] < 1e-2, res
        assert res["arn_x_rel"] < 4e-3 and res["arn_h_rel"] < 8e-3, res
        assert res["dec_prefill_rel"] < 2e-2 and res["dec_tokens_equal"] > 0.9, res
        assert res["ag_rel"] < 1e-2 and res["rs_rel"] < 2e-2, res
        assert abs(res["llama_loss_tp"] - res["llama_loss_full"]) < 3e-2 and res["llama_dw_rel"] < 6e-2, res
        assert res["llama_dnorm_rel"] < 6e-2 and res["llama_dhead_rel"] < 6e-2, res
        assert res["lib_y_rel"] < 3e-2 and res["lib_dx_rel"] < 4e-2 and res["lib_dw_rel"] < 4e-2, res
        assert res["y_rel"] < 3e-2 and res["dx_rel"] < 4e-2 and res["dwc_rel"] < 4e-2 and res["dwr_rel"] < 4e-2 and res["dbr_rel"] < 4e-2, res
