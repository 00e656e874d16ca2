"""The Keras-like layer of the Python binding: ModelBuilder, compile, fit on data loaders, evaluate, predict, summary,
history plots, saving and comparing models."""
import _path  # noqa: F401
import os
import tempfile

import torch

import rustorch as rt

rt.set_seed(0)
X = torch.randn(600, 8)
y = (X[:, 0] * X[:, 1] + X[:, 2] > 0).long()                          # not linearly separable
train = rt.DataLoader(rt.TensorDataset(X[:480], y[:480]), batch_size=32, shuffle=True)
val = rt.DataLoader(rt.TensorDataset(X[480:], y[480:]), batch_size=64)

b = rt.ModelBuilder()
b.dense(32, "relu")
b.dropout(0.05)
b.dense(16, "tanh")
b.dense(2)
model = b.build("xor-ish")
model.compile("adam", "cross_entropy", ["accuracy"], lr=0.01)
hist = model.fit(train, val, epochs=15, verbose=False)
print(model.summary())
print(hist.summary())
print("evaluate:", {k: round(v, 4) for k, v in model.evaluate(val).items()})
print("predict on a Variable ->", type(model.predict(rt.Variable(X[:3]))).__name__)
out = tempfile.mkdtemp()
rt.Plotter().plot_training_history(hist, os.path.join(out, "loss.svg"))
rt.ModelSerializer.export(model, os.path.join(out, "model.safetensors"), "safetensors")
print("saved:", sorted(os.listdir(out)), rt.ModelSerializer.get_model_info(os.path.join(out, "model.safetensors"))["parameters"], "parameters")
twin = b.build("twin")
twin.compile("adam", "cross_entropy")
twin(X[:1])
print("twin before loading:", rt.ModelComparator.compare(model, twin)["parameters_identical"], end="; ")
rt.ModelSerializer.load(twin, os.path.join(out, "model.safetensors"))
print("after:", rt.ModelComparator.compare(model, twin)["parameters_identical"])
