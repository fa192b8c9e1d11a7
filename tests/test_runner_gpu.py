"""The graph-held layer (``moe.Runner``): a replay equals the eager layer on the same rows, for rows on either side of
the one-launch selection threshold, and the host-bound replay (copies as graph nodes) returns the same bits."""

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("direct", [True, False])
@pytest.mark.parametrize("rows", [5, 32, 33, 70])
def test_replay_equals_eager_and_host_bound(rows, direct, pdl):
    from tensorfold_b200 import experts, moe, synthetic

    dev = torch.device("cuda", 0)
    shape = synthetic.SMALL
    gate, up, down = synthetic.affine_layer(shape, dev)
    layer = moe.Routed(synthetic.router_rows(shape, dev), experts.make([gate, up], down, 64), shape.top_k,
                       shared=shape.shared)
    runner = moe.Runner(layer, rows)
    x_host = torch.empty((rows, shape.dims), dtype=torch.bfloat16).pin_memory()
    out_host = torch.zeros((rows, shape.dims), dtype=torch.bfloat16).pin_memory()
    runner.bind_host(x_host, out_host, direct=direct)
    for index in (11, 12):                                  # the replays follow the new rows' experts
        x = synthetic.activations(shape, rows, dev, index=index)
        want = moe.run(x, layer)
        got = runner(x).clone()
        assert torch.equal(got, want)
        x_host.copy_(x.cpu())
        out_host.zero_()
        runner.replay_host()
        torch.cuda.current_stream().synchronize()
        assert torch.equal(out_host, want.cpu())


def test_host_buffers_must_be_pinned():
    from tensorfold_b200 import experts, moe, synthetic

    dev = torch.device("cuda", 0)
    shape = synthetic.SMALL
    gate, up, down = synthetic.affine_layer(shape, dev)
    layer = moe.Routed(synthetic.router_rows(shape, dev), experts.make([gate, up], down, 64), shape.top_k,
                       shared=shape.shared)
    runner = moe.Runner(layer, 4)
    with pytest.raises(ValueError):
        runner.bind_host(torch.empty((4, shape.dims), dtype=torch.bfloat16),
                         torch.empty((4, shape.dims), dtype=torch.bfloat16))
