"""The pinned-staging upload: every byte arrives, whatever the sizes of the
tensors against the staging buffers."""

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
