"""`TensorV2` / `DType` / `Device` / `ops_v2` mirror.  The host-only cases follow the reference's own unit tests
(src/tensor_v2.rs:353-382, src/ops_v2/basic.rs:126-148, src/ops_v2/matmul.rs:52-72); the arithmetic cases need a GPU."""
import numpy as np
import pytest

import rustygradients_b200 as rg
from rustygradients_b200.tensor_v2 import Device, DType, TensorV2, add_op, matmul_op, mul_op, sub_op


def test_tensor_creation_on_the_host():
    t = TensorV2.zeros([2, 3], True, Device.cpu())           # tensor_v2.rs: test_tensor_creation
    assert t.shape() == [2, 3] and t.requires_grad() and t.dtype() is DType.F32
    assert t.device() == Device.cpu() and t.device().device_type() == ("cpu",)
    assert t.grad() is None
    assert [d.name for d in DType] == ["F32", "F16", "BF16", "I32", "U32"]
    o = TensorV2.ones([2, 2], False, Device.cpu())
    assert np.array_equal(o.to_cpu_data(), np.ones((2, 2), np.float32))
    r = TensorV2.randn([3, 4], False)
    assert r.shape() == [3, 4] and not r.requires_grad()
    f = TensorV2.from_slice([2.0, 3.0], [2], False)
    assert f.shape() == [2]
    with pytest.raises(rg.ShapeError):
        TensorV2.from_slice([1.0, 2.0, 3.0], [2, 2], False)
    assert f == f and f != TensorV2.from_slice([2.0, 3.0], [2], False)     # identity of the data, not of the values
    assert "shape: [2]" in repr(f) and "requires_grad: false" in repr(f)


def test_host_tensors_do_not_compute():
    a = TensorV2.ones([2, 2], False, Device.cpu())
    with pytest.raises(rg.Unsupported):
        a.add(a)
    with pytest.raises(rg.Unsupported):
        matmul_op(a, a)


@pytest.mark.gpu
def test_operations_on_the_device():
    dev = Device.cuda(0)
    assert dev.device_type() == ("cuda", 0) and Device.default_device() == dev
    a = TensorV2.ones([2, 2], False, dev)
    b = TensorV2.ones([2, 2], True, dev)
    c = add_op(a, b)                                           # ops_v2/basic.rs: test_add_forward
    assert c.shape() == [2, 2] and c.requires_grad() and np.array_equal(c.to_cpu_data(), np.full((2, 2), 2, np.float32))
    m = mul_op(TensorV2.from_slice([2.0, 3.0], [2], False).to_device(dev), TensorV2.from_slice([4.0, 5.0], [2], False).to_device(dev))
    assert m.shape() == [2] and np.array_equal(m.to_cpu_data(), np.array([8, 15], np.float32))   # test_mul_forward
    assert np.array_equal(sub_op(c, a).to_cpu_data(), np.ones((2, 2), np.float32))
    rng = np.random.default_rng(0)
    x, y = rng.standard_normal((3, 4)).astype(np.float32), rng.standard_normal((4, 5)).astype(np.float32)
    z = matmul_op(TensorV2.new(x, False, dev), TensorV2.new(y, False, dev))                        # test_matmul_2d
    assert z.shape() == [3, 5] and np.abs(z.to_cpu_data() - x.astype(np.float64) @ y).max() < 1e-5
    xb, yb = rng.standard_normal((2, 3, 4)).astype(np.float32), rng.standard_normal((2, 4, 5)).astype(np.float32)
    zb = TensorV2.new(xb, False, dev).matmul(TensorV2.new(yb, False, dev))                         # test_matmul_batched
    assert zb.shape() == [2, 3, 5] and np.abs(zb.to_cpu_data() - xb.astype(np.float64) @ yb).max() < 1e-5
    t = TensorV2.new(x, True, dev)
    assert np.array_equal(t.relu().to_cpu_data(), np.maximum(x, 0)) and t.relu().requires_grad()
    e = np.exp(x - x.max(-1, keepdims=True))
    assert np.abs(t.softmax().to_cpu_data() - e / e.sum(-1, keepdims=True)).max() < 1e-6
    assert np.array_equal(t.reshape([2, 6]).to_cpu_data(), x.reshape(2, 6))
    assert np.array_equal(t.transpose(0, 1).to_cpu_data(), x.T)
    back = t.to_device(Device.cpu())
    assert back.device() == Device.cpu() and np.array_equal(back.to_cpu_data(), x)
    with pytest.raises(rg.Unsupported):
        t.add(back)                                            # operands on different devices
