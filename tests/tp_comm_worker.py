"""Worker of the multi-GPU communication tests (torchrun, one rank per GPU): exercises the peer-memory
primitives one by one and writes a progress log per rank, so a stall can be located from the log."""
import os
import sys
import time

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from ksanallm_b200.ops import native, reference as ref  # noqa: E402
from ksanallm_b200.ops.dispatch import LinearWeight  # noqa: E402
from ksanallm_b200.parallel.symm import ONE_SHOT_ROWS, SymmetricComm  # noqa: E402


def main():
    out_dir = sys.argv[1]
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    log = open(os.path.join(out_dir, f"tp_comm_rank{rank}.log"), "w")

    def say(*a):
        log.write(" ".join(str(x) for x in a) + "\n")
        log.flush()

    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    say("pg ready")
    H, MAXT = 1024, 512
    comm = SymmetricComm(dist.group.WORLD, rank, world, dev, max_tokens=MAXT, hidden=H)
    say("symmetric buffer ready", comm.total)
    comm.barrier()
    torch.cuda.synchronize()
    native.check_err_flag(dev)
    say("barrier ok")
    torch.manual_seed(100 + rank)
    x = torch.randn(64, H, device=dev, dtype=torch.bfloat16)
    want = x.float().clone()
    dist.all_reduce(want)
    got = comm.all_reduce(x)
    torch.cuda.synchronize()
    native.check_err_flag(dev)
    err = float((got.float() - want).abs().max())
    say("all_reduce max err", err)
    assert err < 0.1
    say("multicast address", hex(comm.mc_ptr))
    if comm.mc_ptr:
        res = torch.randn(64, H, device=dev, dtype=torch.bfloat16)
        got = comm.all_reduce(x, residual=res, nvls=True)       # in-switch reduction (multimem.ld_reduce)
        torch.cuda.synchronize()
        native.check_err_flag(dev)
        err = float((got.float() - (want + res.float())).abs().max())
        say("nvls all_reduce max err", err)
        assert err < 0.15
    results = {}
    for M in (4, 16, 64, 200, 500):
        for quant in (False, True):
            torch.manual_seed(7)
            K = 2048
            w_full = torch.randn(H, K * world, device=dev) * 0.05
            x_full = torch.randn(M, K * world, device=dev, dtype=torch.bfloat16)
            h0 = torch.randn(M, H, device=dev, dtype=torch.bfloat16)
            nw = torch.randn(H, device=dev, dtype=torch.bfloat16)
            w = w_full[:, rank * K:(rank + 1) * K].contiguous()
            xs = x_full[:, rank * K:(rank + 1) * K].contiguous()
            W = LinearWeight(w=w.to(torch.bfloat16))
            if quant:
                W = LinearWeight(*([None, None] + list(ref.quant_weight_fp8_block(w))))
            nxt = LinearWeight(wq=torch.empty(8, H, device=dev, dtype=torch.float8_e4m3fn), ws=torch.empty(1, 8, device=dev)) if quant else None
            for rep in range(3):
                comm.begin_forward()
                if not comm.one_shot(M):
                    h = comm.h[:M]
                    h.copy_(h0)
                else:
                    h = h0.clone()
                h, y = comm.row_parallel_norm(xs, W, h, nw, None, 1e-5, False, quant_for=nxt, gather_h=True)
                torch.cuda.synchronize()
                native.check_err_flag(dev)
            # oracle: full product of the (de)quantised operands + residual, then RMSNorm
            part = ref.gemm(xs, W.dense().to(torch.bfloat16) if not quant else W.dense(), out_dtype=torch.float32) if not quant else \
                ref.gemm_fp8(*ref.quant_fp8(xs), W.wq, W.ws, out_dtype=torch.float32)
            total = part.clone()
            dist.all_reduce(total)
            h_want = (total + h0.float()).to(torch.bfloat16)
            y_want = ref.norm(h_want, nw, 1e-5)[0]
            e_h = float((h.float() - h_want.float()).norm() / h_want.float().norm())
            if quant:
                yq, ys = y.q.float(), y.s
                yd = yq.reshape(M, H // 128, 128) * ys[: H // 128, :M].t().unsqueeze(-1)
                e_y = float((yd.reshape(M, H) - y_want.float()).norm() / y_want.float().norm())
            else:
                e_y = float((y.float() - y_want.float()).norm() / y_want.float().norm())
            say(f"row_parallel_norm M={M} quant={quant}: rel err h {e_h:.4f} y {e_y:.4f}")
            results[(M, quant)] = (e_h, e_y)
            assert e_h < 2e-2 and e_y < (8e-2 if quant else 2e-2)
    # column all-gather (logits shards)
    shard = torch.randn(5, 1000, device=dev, dtype=torch.float32) + rank
    gathered = comm.all_gather_cols(shard, 996)
    parts = [torch.empty_like(shard) for _ in range(world)]
    dist.all_gather(parts, shard)
    torch.cuda.synchronize()
    assert torch.equal(gathered, torch.cat([p[:, :996] for p in parts], 1))
    say("all_gather_cols ok")
    # device-timed comparison with the library path on a decode-sized and a prefill-sized case
    for M in (8, 2048 if MAXT >= 2048 else 512):
        K = 1024
        w = (torch.randn(H, K, device=dev) * 0.05).to(torch.bfloat16)
        xs = torch.randn(M, K, device=dev, dtype=torch.bfloat16)
        nw = torch.ones(H, device=dev, dtype=torch.bfloat16)
        W = LinearWeight(w=w)
        hbuf = comm.h[:M] if not comm.one_shot(M) else torch.zeros(M, H, device=dev, dtype=torch.bfloat16)

        def fused():
            comm.begin_forward()
            comm.row_parallel_norm(xs, W, hbuf, nw, None, 1e-5, False)
            comm.row_parallel_norm(xs, W, hbuf, nw, None, 1e-5, False)

        def lib():
            for _ in range(2):
                p = native.gemm_bf16(xs, w)
                dist.all_reduce(p)
                hh = native.add(hbuf, p)
                native.norm(hh, nw, 1e-5)

        for name, fn in (("fused", fused), ("nccl", lib)):
            for _ in range(5):
                fn()
            torch.cuda.synchronize(); dist.barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(20):
                fn()
            e1.record(); torch.cuda.synchronize()
            t = torch.tensor([e0.elapsed_time(e1) / 40], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            say(f"time per row-parallel linear+norm M={M} {name}: {float(t) * 1e3:.1f} us (max over ranks)")
    native.check_err_flag(dev)
    say("done")
    dist.barrier()
    log.close()
    os._exit(0)


if __name__ == "__main__":
    main()
