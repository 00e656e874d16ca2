"""Model compression: post-training int8 / int4 quantisation with calibration, quantisation-aware training, magnitude
and 2:4 pruning with lottery-ticket rewinding, sparse layers."""
import _path  # noqa: F401

import torch

from rustorch_b200 import nn, quantization as Q, sparse as S

torch.manual_seed(0)
w = torch.randn(64, 128)
for name, cfg in (("int8 per tensor", Q.QuantizationConfig()), ("int8 per channel", Q.QuantizationConfig(scheme=Q.QuantizationScheme.PER_CHANNEL_SYMMETRIC)),
                  ("int4", Q.QuantizationConfig(qtype=Q.QuantizationType.INT4))):
    q = Q.quantize_tensor(w, cfg)
    print(f"{name:<17} max error {float((q.dequantize() - w).abs().max()):.4f}")
outlier = torch.randn(20000)
outlier[0] = 80.0
for name, mode in (("min/max", nn.CalibrationMode.MIN_MAX), ("99.9 percentile", nn.CalibrationMode.percentile(0.999)), ("entropy", nn.CalibrationMode.ENTROPY)):
    t = nn.Quantizer(mode, True).quantize_tensor(outlier, nn.QuantizationType.INT8)
    print(f"calibration {name:<16} rms error on the bulk {float((t.dequantize()[1:] - outlier[1:]).pow(2).mean().sqrt()):.4f}")
a, b = torch.randn(16, 32), torch.randn(32, 8)
print("int8 matmul error: %.3f" % float((Q.QuantizedOps.qmatmul(Q.quantize_tensor(a), Q.quantize_tensor(b)).dequantize() - a @ b).abs().max()))

X, y = torch.randn(256, 16), torch.randn(256, 1)
qat = nn.QuantizationAwareModule(nn.Sequential(nn.Linear(16, 32), nn.ReLU(), nn.Linear(32, 1)), weights=True)
qat.enable_qat()
opt = torch.optim.Adam(qat.parameters(), 1e-2)
for _ in range(100):
    opt.zero_grad()
    loss = torch.nn.functional.mse_loss(qat(X), y)
    loss.backward()
    opt.step()
print("quantisation-aware training loss: %.4f (input scale %.4f)" % (float(loss.detach()), qat.qparams["input"].scale))

net = nn.Sequential(nn.Linear(16, 32), nn.ReLU(), nn.Linear(32, 1))
pruner = nn.Pruner(nn.PruningMethod.L1_NORM, nn.PruningStructure.UNSTRUCTURED, 0.8, nn.PruningSchedule.polynomial(0, 4, 3.0))
wrapped = nn.PruningAwareModule(net, pruner)
wrapped.enable_pruning()
opt = torch.optim.Adam(wrapped.parameters(), 1e-2)
for epoch in range(6):
    for _ in range(30):
        opt.zero_grad()
        loss = torch.nn.functional.mse_loss(wrapped(X), y)
        loss.backward()
        opt.step()
    wrapped.step_epoch()
    print(f"epoch {epoch}: target sparsity {pruner.current_sparsity():.2f}  actual {pruner.get_global_sparsity():.2f}  loss {float(loss.detach()):.4f}")
pruner.rewind(net.named_parameters())
print("rewound to the initial weights under the final mask; zeros kept: %.2f" % float((net[0].weight == 0).float().mean()))
two_four = nn.Pruner(nn.PruningMethod.L1_NORM, nn.PruningStructure.block(2, 4), 0.5, nn.PruningSchedule.ONE_SHOT).compute_mask(w)
print("2:4 mask keeps exactly two of every four:", bool((two_four.view(-1, 4).sum(1) == 2).all()))
sl = S.SparseLinear.from_dense(torch.nn.Linear(128, 64), 0.9)
print("SparseLinear (CSR) sparsity %.2f, output" % sl.sparsity(), tuple(sl(torch.randn(4, 128)).shape))
