"""safetensors wire format: our writer/reader against the `safetensors` package
(CPU), and a device round trip of parameters + Adam state (GPU)."""
import numpy as np
import pytest

from zigrad_b200 import checkpoint


def test_wire_format_agrees_with_the_safetensors_package(tmp_path):
    st = pytest.importorskip("safetensors.numpy")
    g = np.random.Generator(np.random.PCG64(1))
    tensors = {"layers.0.weight": g.standard_normal((5, 7)).astype(np.float32), "layers.0.bias": g.standard_normal(5).astype(np.float32),
               "adam.t": np.array([12], np.uint64), "empty": np.zeros((0, 3), np.float32), "d": g.standard_normal((2, 2, 2))}
    blob = checkpoint.serialize(tensors, {"k": "v"})
    theirs = st.load(blob)
    assert set(theirs) == set(tensors)
    for k in tensors:
        np.testing.assert_array_equal(theirs[k], tensors[k])
        assert theirs[k].dtype == tensors[k].dtype
    ours = checkpoint.deserialize(st.save(tensors, {"k": "v"}))
    for k in tensors:
        np.testing.assert_array_equal(ours[k], tensors[k])
    assert checkpoint.metadata(blob) == {"k": "v"}
    with pytest.raises(ValueError):
        checkpoint.deserialize(blob[:4])


@pytest.mark.gpu
def test_mlp_checkpoint_round_trip_resumes_bit_identically(gpu, tmp_path):
    from zigrad_b200.mlp import MlpTrainer, kaiming_uniform
    dims, B = [32, 24, 16, 5], 64
    g = np.random.Generator(np.random.PCG64(3))
    Ws, bs = kaiming_uniform(dims, 2)
    X = g.uniform(0, 1, (B, dims[0])).astype(np.float32)
    T = np.eye(dims[-1], dtype=np.float32)[g.integers(0, dims[-1], B)]
    Xd, Td = gpu.from_numpy(X), gpu.from_numpy(T)
    a = MlpTrainer(gpu, dims, B, Ws, bs, "adam", lr=1e-2, clip=True)
    for _ in range(3):
        a.step(Xd, Td)
    path = str(tmp_path / "ckpt.safetensors")
    checkpoint.save_mlp(a, path)
    b = MlpTrainer(gpu, dims, B, [np.zeros_like(w) for w in Ws], [np.zeros_like(x) for x in bs], "adam", lr=1e-2, clip=True)
    checkpoint.load_mlp(b, path)
    assert b.read_t() == a.read_t() == 18
    for _ in range(2):  # same state, same inputs: the two trainers stay equal (up to the order of fp32 atomics in split-K)
        a.step(Xd, Td)
        b.step(Xd, Td)
    pa, pb = gpu.to_numpy(a.params), gpu.to_numpy(b.params)
    np.testing.assert_allclose(pb, pa, rtol=1e-5, atol=1e-7)
    assert abs(a.read_loss() - b.read_loss()) <= 1e-6 * abs(a.read_loss())
    a.free()
    b.free()
