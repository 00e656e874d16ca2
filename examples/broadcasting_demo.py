"""Broadcasting rules: which shapes combine, explicit expansion (shared vs owned), bias addition."""
import _path  # noqa: F401

import rustorch as rt

batch = rt.Tensor.ones([4, 3])
bias = rt.tensor([0.1, 0.2, 0.3])
col = rt.tensor([[1.0], [2.0], [3.0], [4.0]])
for name, other in (("bias [3]", bias), ("column [4, 1]", col), ("mismatch [4]", rt.Tensor.ones([4]))):
    print(f"[4, 3] with {name}: can broadcast = {batch.can_broadcast_with(other)}")
print("batch + bias  :", (batch + bias).as_slice()[:3])
print("batch * column:", (batch * col).as_slice()[::3])
view = bias.unsqueeze(0).expand_shared([4, 3])
own = bias.unsqueeze(0).expand_owned([4, 3])
print("expand_shared strides", tuple(view.data.stride()), "(no copy); expand_owned strides", tuple(own.data.stride()))
print("outer product by broadcasting:", (col * bias.unsqueeze(0)).shape)
