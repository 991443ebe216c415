"""The launchers inside a CUDA graph.

Every entry point only enqueues work on the stream it is given (no synchronisation, no
allocation on the way), so a sequence of them can be captured once and replayed, which is
how a launch-bound loop of small kernels is run.  The test captures one call of each
kernel, replays the graph on new input contents and requires the replay to equal the
eager result bit for bit (same kernels, same arithmetic).

A matmul with too few tiles for the device normally takes the split along K, whose scratch
array is allocated at the first such launch on a stream.  Allocation is not possible while
a stream is being captured: a first launch inside a capture must fall back to the ordinary
kernel, and still be correct.
"""

import pytest
import torch

from gpu_util import assert_device_healthy

pytestmark = pytest.mark.gpu


def make_inputs(seed):
    g = torch.Generator(device="cuda").manual_seed(seed)

    def normal(*shape):
        return torch.randn(*shape, generator=g, device="cuda").half()

    return {
        "c": normal(512, 768), "a": normal(512, 320), "b": normal(320, 768),
        "a_long": normal(256, 8192), "b_long": normal(8192, 256),
        "x": (4 * normal(300, 1000)),
        "q": normal(1, 2, 256, 128), "k": normal(1, 2, 256, 128), "v": normal(1, 2, 256, 128),
        "image": normal(2, 16, 12, 12), "filter": normal(24, 16, 3, 3) / 12,
    }


def make_outputs():
    def empty(*shape):
        return torch.empty(*shape, dtype=torch.float16, device="cuda")

    return {"addmm": empty(512, 768), "long": empty(256, 256), "softmax": empty(300, 1000),
            "attention": empty(1, 2, 256, 128), "conv2d": empty(2, 24, 12, 12), "pool": empty(2, 24, 6, 6)}


def run_all(i, o, workspace):
    from ninetoothed_b200 import _capi

    _capi.addmm(i["c"], i["a"], i["b"], 0.5, 2.0, o["addmm"])
    _capi.matmul(i["a_long"], i["b_long"], o["long"])
    _capi.softmax(i["x"], o["softmax"])
    _capi.attention(i["q"], i["k"], i["v"], True, o["attention"], scale=0.088)
    _capi.conv2d(i["image"], i["filter"], o["conv2d"], 1, 1, workspace=workspace)
    _capi.max_pool2d(o["conv2d"], o["pool"], 2, 2, False)


@pytest.mark.parametrize("warm", [True, False])
def test_capture_and_replay_match_eager(warm):
    """warm: the capture stream has run every kernel before (scratch exists, the long matmul is split);
    otherwise the first launches on that stream happen inside the capture."""
    from ninetoothed_b200 import _capi

    _capi.device_status()  # the per-device state (one small allocation) is made at the first call: not inside a capture
    static_in, static_out = make_inputs(1), make_outputs()
    workspace = torch.empty(max(_capi.conv2d_workspace_size(static_in["image"], static_in["filter"]), 1),
                            dtype=torch.uint8, device="cuda")
    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    if warm:
        with torch.cuda.stream(stream):
            run_all(static_in, static_out, workspace)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(stream):
        with torch.cuda.graph(graph, stream=stream):
            run_all(static_in, static_out, workspace)
    torch.cuda.current_stream().wait_stream(stream)
    torch.cuda.synchronize()

    for seed in (2, 3):
        fresh = make_inputs(seed)
        for name, tensor in fresh.items():
            static_in[name].copy_(tensor)
        for tensor in static_out.values():
            tensor.fill_(float("nan"))
        graph.replay()
        torch.cuda.synchronize()
        eager_out = make_outputs()
        run_all(fresh, eager_out, workspace)
        torch.cuda.synchronize()
        for name in eager_out:
            assert torch.isfinite(static_out[name]).all(), name
            if name == "long" and not warm:
                # eager splits along K, the capture could not: other summation order, same tolerance as elsewhere
                torch.testing.assert_close(static_out[name].float(), eager_out[name].float(), rtol=1e-2, atol=1e-2)
            else:
                assert torch.equal(static_out[name], eager_out[name]), name
    reference = (fresh["a_long"].float() @ fresh["b_long"].float()).half()
    torch.testing.assert_close(static_out["long"].float(), reference.float(), rtol=1e-2, atol=1e-1)
    assert_device_healthy()
