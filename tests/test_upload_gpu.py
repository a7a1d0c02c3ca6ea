"""The pinned-staging upload: every byte arrives, whatever the sizes of the
tensors against the staging buffers."""

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


@pytest.mark.parametrize("staging,buffers,threads", [(1000, 2, 1), (4096, 3, 2), (64 << 20, 3, 4)])
def test_upload_keeps_every_byte(staging, buffers, threads):
    from reflex_b200.weights.upload import Uploader, upload_all

    g = torch.Generator().manual_seed(staging)
    host = {
        "matrix": torch.randn(123, 77, generator=g).bfloat16(),
        "norm": torch.randn(333, generator=g),
        "one": torch.randn(1, generator=g),
        "none": torch.empty(0, 5),
        "table": torch.randint(0, 1000, (7, 9), generator=g, dtype=torch.int32),
        "strided": torch.randn(40, 50, generator=g)[:, ::2],           # not contiguous
        "large": torch.randn(3_000_017, generator=g).bfloat16(),         # several buffers, odd size
    }
    out = upload_all(host, DEV, staging_bytes=staging, buffers=buffers, threads=threads)
    assert list(out) == list(host)
    for name, t in host.items():
        d = out[name]
        assert d.device.type == "cuda" and d.dtype == t.dtype and d.shape == t.shape
        assert torch.equal(d.cpu(), t), name
    # an uploader is reusable tensor after tensor, and counts what it moved
    up = Uploader(DEV, staging_bytes=staging, buffers=buffers, threads=threads)
    a = up.upload(host["large"])
    b = up.upload(host["matrix"])
    up.finish()
    assert torch.equal(a.cpu(), host["large"]) and torch.equal(b.cpu(), host["matrix"])
    assert up.bytes_copied == host["large"].numel() * 2 + host["matrix"].numel() * 2


def test_upload_refuses_bad_settings():
    from reflex_b200.weights.upload import Uploader

    with pytest.raises(ValueError):
        Uploader("cpu")
    with pytest.raises(ValueError):
        Uploader(DEV, buffers=1)


@pytest.mark.parametrize("shape,role", [((1000, 96), "matrix"), ((4097,), "norm"), ((3, 5, 7), "matrix"),
                                        ((151936, 128), "table")])
def test_random_weights_are_the_same_on_the_host_and_on_the_device(shape, role):
    """The counter-based draw gives the same bits from the CUDA kernel and from
    the NumPy restatement, in both element types, so a model drawn on the GPU
    (the benchmark's) can be rebuilt tensor by tensor on the CPU."""
    from reflex_b200.weights.random_init import draw, draw_host, tensor_key

    name = f"model.layers.3.x.{role}"
    for dtype in (torch.float32, torch.bfloat16):
        dev = draw(name, shape, role, 11, "cuda:0", dtype)
        kind, a, b = ("uniform", 0.9, 1.1) if role == "norm" else ("normal", 0.0, 0.02)
        n = int(np.prod(shape))
        host = torch.from_numpy(draw_host(tensor_key(11, name), n, kind, a, b)).reshape(shape).to(dtype)
        assert torch.equal(dev.cpu(), host)
