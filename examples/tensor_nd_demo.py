"""N-dimensional tensors: construction, shape operations, reductions, indexing helpers."""
import _path  # noqa: F401

import rustorch as rt

t = rt.Tensor.arange(0, 24).reshape([2, 3, 4])
print("shape", t.shape, "ndim", t.ndim, "numel", t.numel)
print("sum over axis 2:", t.sum_axis(2).as_slice())
print("transpose(0, 2):", t.transpose(0, 2).shape, " flatten_from(1):", t.flatten_from(1).shape)
print("unsqueeze_multiple([0, 4]):", t.unsqueeze_multiple([0, 4]).shape, " squeeze_all:", t.unsqueeze(0).squeeze_all().shape)
print("mean %.2f  std %.3f  median-ish %.1f" % (float(t.mean()), t.std_unbiased(), t.quantile_advanced(0.5)))
print("values > 20 at flat indices", t.find_all(lambda x: x > 20), "; count of even values", t.count_where(lambda x: x % 2 == 0))
rolled = rt.tensor([1.0, 2.0, 3.0, 4.0]).roll_1d(1, 0)
print("roll_1d:", rolled.as_slice(), " repeat_advanced:", rt.tensor([[1.0, 2.0]]).repeat_advanced([2, 2]).as_slice())
a, b = rt.Tensor.eye(3), rt.Tensor.full([3, 3], 2.0)
print("eye @ full:", a.matmul(b).as_slice()[:3], " stack:", rt.Tensor.stack([a, b]).shape)
