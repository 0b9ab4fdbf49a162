"""A tensor on a GPU that is not the current device must be refused before anything is launched:
the library launches on the current device's stream, so another GPU's pointers would fault there."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2,
                    reason="needs two visible GPUs")
def test_tensor_on_another_device_is_rejected_before_any_launch():
    from better_benchmark_b200 import kernels, native

    lib = native.load()
    torch.cuda.set_device(0)
    x = torch.randn(64, 256, device="cuda:1")
    before = lib.b200_launch_count()
    with pytest.raises(native.KernelArgumentError, match="current device"):
        kernels.row_reduce(x, "sum")
    with pytest.raises(native.KernelArgumentError, match="current device"):
        kernels.softmax(x)
    assert lib.b200_launch_count() == before
    with torch.cuda.device(1):
        out = kernels.row_reduce(x, "sum")
    assert torch.allclose(out.cpu(), x.cpu().sum(-1), atol=1e-4)


def test_scratch_buffer_never_releases_a_superseded_buffer():
    from better_benchmark_b200 import kernels

    dev = torch.device("cuda", torch.cuda.current_device())
    first = kernels.scratch_buffer(dev, 1024)
    ptr = first.data_ptr()
    bigger = kernels.scratch_buffer(dev, first.numel() + 4096)
    assert bigger.numel() >= first.numel() + 4096
    held = kernels._scratch_by_device[kernels._device_key(dev)]
    assert any(b.data_ptr() == ptr for b in held), "the earlier buffer must stay alive for captured graphs"
    g = torch.cuda.CUDAGraph()
    with pytest.raises(RuntimeError, match="grow"):
        with torch.cuda.graph(g):
            kernels.scratch_buffer(dev, bigger.numel() * 2)
