"""Plots as SVG text and graphs as Graphviz text: training curves, tensors, attention maps, the autograd graph."""
import _path  # noqa: F401
import os
import tempfile

import torch

import rustorch as rt
from rustorch_b200 import visualization as Z

out = tempfile.mkdtemp()
hist = rt.TrainingHistory()
for e in range(12):
    hist.add_epoch(1.0 / (e + 1) + 0.05, 1.2 / (e + 1) + 0.1, {"accuracy": 1 - 0.5 / (e + 1)})
pl = rt.Plotter(figure_size=(8, 4))
pl.plot_training_history(hist, os.path.join(out, "history.svg"))
pl.line_plot(list(range(20)), [x ** 0.5 for x in range(20)], "square root", "x", "sqrt(x)", os.path.join(out, "line.svg"))
pl.scatter_plot(torch.randn(50).tolist(), torch.randn(50).tolist(), colors=torch.rand(50).tolist(), save_path=os.path.join(out, "scatter.svg"))
pl.histogram(torch.randn(1000).tolist(), 25, "normal samples", save_path=os.path.join(out, "hist.svg"))
pl.plot_tensor_as_image(torch.randn(12, 16), "weights", save_path=os.path.join(out, "tensor.svg"))
mv = rt.ModelVisualizer()
att = torch.softmax(torch.randn(4, 5, 5), -1)
mv.plot_attention_heatmap(att, ["the", "cat", "sat", "down", "."], "head average", os.path.join(out, "attention.svg"))
net = torch.nn.Sequential(torch.nn.Linear(4, 8), torch.nn.Tanh(), torch.nn.Linear(8, 1))
open(os.path.join(out, "modules.dot"), "w").write(mv.visualize_model(net))
x = torch.randn(2, 4, requires_grad=True)
open(os.path.join(out, "autograd.dot"), "w").write(Z.GraphVisualizer().autograd_dot(net(x).sum()))
dash = Z.create_dashboard([("history", open(os.path.join(out, "history.svg")).read()), ("weights", open(os.path.join(out, "tensor.svg")).read())])
open(os.path.join(out, "dashboard.html"), "w").write(dash)
ts = rt.TensorStats(torch.randn(1000))
ts.compute_stats()
print("files:", sorted(os.listdir(out)))
print("tensor statistics:", {k: round(v, 3) for k, v in ts.get_stats().items()})
