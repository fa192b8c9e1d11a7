"""Expert parallelism on two GPUs over NCCL: every token's output equals the one-GPU layer's, bit for bit (the same
kernels run on each pair, the home rank sums in slot order).  Needs two devices; skipped otherwise."""

import os
import socket
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def _worker(rank, world, port, out):
    sys.path.insert(0, str(ROOT))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist

    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    from tensorfold_b200 import ep, experts, moe, synthetic

    shape, rows = synthetic.SMALL, 20
    per = shape.experts // world
    gate, up, down = synthetic.affine_layer(shape, dev)
    router = synthetic.router_rows(shape, dev)
    sl = slice(rank * per, (rank + 1) * per)
    local = experts.make([tuple(t[sl].contiguous() for t in gate), tuple(t[sl].contiguous() for t in up)],
                         tuple(t[sl].contiguous() for t in down), 64)
    layer = ep.ExpertParallel(ep.CudaBackend(router, local, shape.top_k, shape.experts), shape.experts, shape.top_k,
                              False)
    x = synthetic.activations(shape, rows, dev, index=50 + rank)
    got = layer.forward(x)
    full = moe.Routed(router, experts.make([gate, up], down, 64), shape.top_k, shared=False)
    want = moe.run(x, full)
    gathered = ep.GatheredExpertParallel(router, local, shape.experts, shape.top_k, rows)
    got2 = gathered.forward(x).clone()
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        gathered.forward(x)
    gathered.out.zero_()
    graph.replay()
    torch.cuda.synchronize()
    fast = ep.GatheredExpertParallel(router, local, shape.experts, shape.top_k, rows, reduce="tokens")
    got3 = fast.forward(x).float()
    close = bool(((got3 - want.float()).norm() / want.float().norm()) < 1e-2)
    flags = (bool(torch.equal(got, want)), bool(torch.equal(got2, want)), bool(torch.equal(gathered.out, want)), close)
    del graph
    torch.cuda.synchronize()
    out.put((rank, flags))
    dist.barrier()
    dist.destroy_process_group()


def _peer_worker(rank, world, port, out):
    try:
        _peer_body(rank, world, port, out)
    except Exception as err:                                         # reported instead of a silent queue time-out
        out.put((rank, (False, repr(err))))
        raise


def _peer_body(rank, world, port, out):
    """The peer-memory form: three eager steps (both buffer parities), then two replays of a captured step."""

    sys.path.insert(0, str(ROOT))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist

    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    from tensorfold_b200 import _lib, ep, experts, moe, synthetic

    shape, rows = synthetic.SMALL, 24
    per = shape.experts // world
    gate, up, down = synthetic.affine_layer(shape, dev)
    router = synthetic.router_rows(shape, dev)
    sl = slice(rank * per, (rank + 1) * per)
    local = experts.make([tuple(t[sl].contiguous() for t in gate), tuple(t[sl].contiguous() for t in up)],
                         tuple(t[sl].contiguous() for t in down), 64)
    full = moe.Routed(router, experts.make([gate, up], down, 64), shape.top_k, shared=False)
    nccl = ep.GatheredExpertParallel(router, local, shape.experts, shape.top_k, rows, reduce="tokens")
    peer = ep.PeerExpertParallel(router, local, shape.experts, shape.top_k, rows)
    flags = []
    xs = [synthetic.activations(shape, rows, dev, index=70 + 2 * i + rank) for i in range(5)]
    for x in xs[:3]:
        got = peer.forward(x).clone()
        ref = nccl.forward(x).clone()
        want = moe.run(x, full).float()
        # two ranks: a + b in either order is the same fp32 value, so the NCCL partial-sum form gives the same bits
        flags.append(bool(torch.equal(got, ref)) and bool((got.float() - want).norm() / want.norm() < 1e-2))
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        peer.forward()                                   # the rows are written into the window by the caller
    for x in xs[3:]:
        peer.tokens.copy_(x)
        peer.out.zero_()
        graph.replay()
        torch.cuda.synchronize()
        flags.append(bool(torch.equal(peer.out, nccl.forward(x))))
    del graph
    torch.cuda.synchronize()
    # rows read from and results stored to pinned host memory by the kernels themselves
    x_pin, out_pin = xs[0].cpu().pin_memory(), torch.zeros((rows, shape.dims), dtype=torch.bfloat16).pin_memory()
    peer.forward(x_pin, out_pin)
    torch.cuda.synchronize()
    flags.append(bool(torch.equal(out_pin, nccl.forward(xs[0]).cpu())))

    # a layer with a shared expert: replicated, run on the own rows, joined in the final sum
    sh = synthetic.SMALL_SHARED
    gate, up, down = synthetic.affine_layer(sh, dev)
    router_s = synthetic.router_rows(sh, dev)
    per = sh.experts // world
    sl, last = slice(rank * per, (rank + 1) * per), slice(sh.experts, sh.experts + 1)

    def cut(which):
        return experts.make([tuple(t[which].contiguous() for t in gate), tuple(t[which].contiguous() for t in up)],
                            tuple(t[which].contiguous() for t in down), 64)

    full_s = moe.Routed(router_s, experts.make([gate, up], down, 64), sh.top_k, shared=True)
    peer_s = ep.PeerExpertParallel(router_s, cut(sl), sh.experts, sh.top_k, rows, shared_experts=cut(last))
    for i in range(2):
        x = synthetic.activations(sh, rows, dev, index=90 + 2 * i + rank)
        got = peer_s.forward(x).float()
        want = moe.run(x, full_s).float()
        flags.append(bool((got - want).norm() / want.norm() < 4e-3))

    # EXL3 routed experts: the rank's share through exl3.routed, fp32 out
    from tensorfold_b200.exl3 import experts as x3

    eg, eu, ed = synthetic.exl3_layer(shape, dev, 4)
    ex_full = x3.prepare(eg, eu, ed, x3.CB_3INST, device=dev)
    ex_mine = x3.prepare(eg[sl], eu[sl], ed[sl], x3.CB_3INST, device=dev)
    peer_x = ep.PeerExl3ExpertParallel(router, ex_mine, shape.experts, shape.top_k, rows)

    class _Cfg:
        num_experts_per_tok, num_experts = shape.top_k, shape.experts
        moe_intermediate_size, hidden_size = shape.width, shape.dims

    buf = moe.MoEBuffers(rows, _Cfg, dev, shared=False)
    scratch = x3.Scratch(ex_full, rows, shape.top_k, device=dev)
    for i in range(2):
        x = synthetic.activations(shape, rows, dev, index=95 + 2 * i + rank)
        got = peer_x.forward(x).clone()
        moe.router(x, router, buf.logits)
        moe.select_rows(buf.logits, buf, shape.top_k, shape.experts)
        want = x3.routed(x, buf.pick, buf.wts, ex_full, scratch, None, rows)
        flags.append(bool(torch.isfinite(got).all()) and bool((got - want).norm() / want.norm() < 1e-5))
        # the next hidden state formed by the summing kernel itself: bf16(h + layer(h)), the same bits as the add after it
        nxt = peer_x.forward(x, residual=True)
        flags.append(bool(torch.equal(nxt, (x.float() + got).to(torch.bfloat16))))
    flags.append(_lib.kernel_status() == 0)
    torch.cuda.synchronize()
    out.put((rank, tuple(flags)))
    dist.barrier()
    dist.destroy_process_group()


def _run_two(worker):
    import torch.multiprocessing as mp

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    procs = [ctx.Process(target=worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    results = [out.get(timeout=240) for _ in procs]
    for p in procs:
        p.join(timeout=120)
    return results, [p.exitcode for p in procs]


def test_peer_memory_form_matches_nccl_form():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    results, codes = _run_two(_peer_worker)
    assert all(all(flags) for _, flags in results), results
    assert codes == [0, 0]


def test_two_gpus_match_one():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    results = [out.get(timeout=300) for _ in procs]
    assert all(all(flags) for _, flags in results), results        # (counted all-to-all, gathered, gathered in a graph, partial sums)
    for p in procs:
        p.join(timeout=120)
    assert [p.exitcode for p in procs] == [0, 0]
