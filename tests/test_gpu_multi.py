"""Two-GPU test of the sharded linear: out-feature shards + all-gather, both over NCCL and by
peer stores (``npb_allgather_push``).  Runs only where two CUDA devices are visible; one child
process per GPU."""

import os
import socket

import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, q) -> None:
    import sys
    from pathlib import Path

    root = Path(__file__).resolve().parents[1]
    for p in (root, root / "oracle", root / "tests"):
        sys.path.insert(0, str(p))
    import torch.distributed as dist

    import oracle
    from helpers import assert_output_close
    from neuropress_b200.nn import NPVQLinear, VQProxy
    from neuropress_b200.sharding import ShardedLinear
    from synthetic import make_activations, make_vq_layer

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    ok, msg = True, ""
    try:
        d = make_vq_layer(512, 1024, num_centroids=65536, bits=16, seed=3, residual_centroids=256,
                          row_scale=True, bias=True)
        full = NPVQLinear(VQProxy(d.centroids), d.packed, 16, 512, 1024, 8, backend="auto", bias=d.bias,
                          residual_proxy=VQProxy(d.residual_centroids), residual_indices=d.residual_indices,
                          row_scale=d.row_scale)
        layer = ShardedLinear.from_layer(full, rank, world)
        layer.local.proxy.to(dev)
        layer.local.residual_proxy.to(dev)
        layer.to(dev)
        refs = {}
        for rows in (1, 2, 16, 300):
            x = make_activations(rows, 1024, torch.bfloat16, seed=rows)
            refs[rows] = (x.to(dev), oracle.vq_forward_f32(x, d.packed, d.centroids, 16, 512, 1024, d.bias,
                                                           **d.ext()))
        for rows, (x, ref) in refs.items():           # NCCL all-gather
            y = layer(x)
            assert y.shape == (rows, 512)
            assert_output_close(y, ref, torch.bfloat16)
        layer.enable_push_gather(max_rows=300, dtype=torch.bfloat16, device=dev)
        for it in range(3):                           # fused all-gather, buffers alternate
            for rows, (x, ref) in refs.items():
                y = layer(x)
                assert y.shape == (rows, 512)
                assert_output_close(y, ref, torch.bfloat16)
        for rows, (x, ref) in refs.items():           # stand-alone push kernel
            y = layer.push(layer.local(x))
            assert y.shape == (rows, 512)
            assert_output_close(y, ref, torch.bfloat16)
        # CUDA-graph replay: the launch arguments are constant, the epoch lives on the device
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                outs = [layer(refs[rows][0]) for rows in (2, 300)]   # an even number of calls
            for _ in range(3):
                graph.replay()
            side.synchronize()
        for rows, y in zip((2, 300), outs):
            assert_output_close(y, refs[rows][1], torch.bfloat16)
        assert layer.push.status() == 0

        # outside what the peer-store buffers were built for (more rows than max_rows, another
        # dtype): the layer falls back to the NCCL all-gather instead of raising
        xb = make_activations(400, 1024, torch.bfloat16, seed=400)
        yb = layer(xb.to(dev))
        assert yb.shape == (400, 512)
        assert_output_close(yb, oracle.vq_forward_f32(xb, d.packed, d.centroids, 16, 512, 1024, d.bias, **d.ext()),
                            torch.bfloat16)
        xf = make_activations(2, 1024, torch.float32, seed=7)
        yf = layer(xf.to(dev))
        assert yf.shape == (2, 512) and yf.dtype == torch.float32
        assert_output_close(yf, oracle.vq_forward_f32(xf, d.packed, d.centroids, 16, 512, 1024, d.bias, **d.ext()),
                            torch.float32)
        y2 = layer(refs[2][0])                        # and back inside the envelope
        assert_output_close(y2, refs[2][1], torch.bfloat16)
        assert layer.push.status() == 0

        # a group-affine (HQQ-style) layer through the same fused all-gather
        from neuropress_b200.nn import NPLinear
        from synthetic import make_q_layer

        qd = make_q_layer(512, 1024, group_size=64, asym=True, seed=5, bias=True)
        qfull = NPLinear(qd.codes, qd.scale, 512, 1024, 64, 4, "asym", "auto", bias=qd.bias,
                         zero_point=qd.zero_point)
        qlayer = ShardedLinear.from_layer(qfull, rank, world).to(dev)
        qlayer.push = layer.push          # same output shape: the buffers and flags are shared
        for rows in (1, 8, 16, 300):
            x = make_activations(rows, 1024, torch.bfloat16, seed=rows)
            ref = oracle.q_forward_f64(x, qd.codes, qd.scale, 4, 64, qd.zero_point, qd.bias)
            for _ in range(2):
                y = qlayer(x.to(dev))
                assert y.shape == (rows, 512)
                assert_output_close(y, ref, torch.bfloat16)
        assert qlayer.push.status() == 0
    except Exception as exc:  # report instead of hanging the peer
        import traceback

        traceback.print_exc()
        ok, msg = False, repr(exc)[:500]
    finally:
        q.put((rank, ok, msg))
        try:
            dist.barrier()
        except Exception:
            pass
        dist.destroy_process_group()


def test_sharded_linear_two_gpus():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two CUDA devices")
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = sorted(q.get(timeout=150) for _ in procs)
    for p in procs:
        p.join(timeout=120)
    assert results == [(0, True, ""), (1, True, "")], results
