"""Rank body of tests/test_tp_sharding_cpu.py (a module of its own so that spawned children can import it:
it registers the hyphen-named package directory before anything else)."""
import os
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
import __graft_entry__ as ge  # noqa: E402

ge.package()

import numpy as np  # noqa: E402
import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

from fish_audio_cpp_b200 import stack as S  # noqa: E402
from fish_audio_cpp_b200 import synth  # noqa: E402


def worker(rank, world, port, q):
    from oracle import oracle
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        M, N, K, g = 5, 48, 768, 256          # 3 groups over 2 ranks: 2 + 1
        X, W, ws = synth.linear_case(3, M, N, K, g)
        full = oracle.linear(W, ws, g, X)
        # column-parallel: rows [rank*N/world, ...) — outputs are independent per row
        lo, hi = rank * N // world, (rank + 1) * N // world
        part = torch.from_numpy(oracle.linear(W[lo:hi], ws[lo:hi], g, X).view(np.uint16).astype(np.int32))
        gathered = [torch.empty_like(part) for _ in range(world)]
        dist.all_gather(gathered, part)
        col = np.concatenate([t.numpy().astype(np.uint16) for t in gathered], axis=1).view(np.float16)
        ok_col = bool(np.array_equal(col.view(np.uint16), full.view(np.uint16)))
        # row-parallel: K cut at group boundaries; activation scales are per (token, group) so the local
        # quantiser needs nothing from the other rank
        b = S.shard_bounds(K // g, world)
        k0, k1 = b[rank] * g, b[rank + 1] * g
        Xq, Xs = oracle.quantize(X[:, k0:k1], g)
        fq, fs = oracle.quantize(X, g)
        ok_quant = bool(np.array_equal(Xq, fq[:, k0:k1]) and np.array_equal(Xs, fs[:, b[rank]:b[rank + 1]]))
        _, y32 = oracle.linear_q(np.ascontiguousarray(W[:, k0:k1]), ws.reshape(N, -1)[:, b[rank]:b[rank + 1]], Xq, Xs, g,
                                 want_f32=True)
        t = torch.from_numpy(y32.copy())
        dist.all_reduce(t)
        ulp = oracle.ulp_distance_fp16(t.numpy().astype(np.float16), full).max()
        q.put((rank, ok_col, ok_quant, int(ulp)))
    finally:
        dist.destroy_process_group()




def lm_head_worker(rank, world, port, q):
    """One rank of the column-parallel LM head on CPU: the oracle computes this rank's row range of a small head,
    the slices are gathered (gloo) and must equal the full head bit for bit."""
    from oracle import oracle
    from fish_audio_cpp_b200 import lm_head as lmh
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        M, vocab, K, g = 3, 16 * 13 + 5, 512, 256   # 13 row tiles over 2 ranks (7 + 6) and a ragged tail of 5
        X, W, ws = synth.linear_case(11, M, vocab, K, g)
        full = oracle.linear(W, ws, g, X)
        lo, hi = lmh.vocab_shard(vocab, world, rank)
        # (the fp16 bit patterns travel as int32: gloo has no 16-bit integer all-gather)
        local = torch.from_numpy(oracle.linear(W[lo:hi], ws[lo:hi], g, X).view(np.uint16).astype(np.int32))
        got = lmh.gather_logits(torch, dist, local, vocab, world).numpy()
        q.put((rank, bool(np.array_equal(got, full.view(np.uint16).astype(np.int32))), (lo, hi)))
    finally:
        dist.destroy_process_group()


def top_up_worker(rank, world, port, q):
    """Two benchmark ranks whose clocks disagree on whether the load window is over must still run the same number of
    further steps (a tensor-parallel step that one rank runs alone waits out every exchange)."""
    import bench
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        remaining = [0.2, -0.01][rank]   # rank 1 thinks the window is already over
        step_s = [1e-3, 2e-3][rank]
        q.put((rank, bench.agreed_top_up_steps(torch, dist, remaining, step_s, "cpu"),
               bench.agreed_top_up_steps(torch, dist, -1.0, step_s, "cpu")))
    finally:
        dist.destroy_process_group()


def free_port():
    import socket
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def gpu_exchange_worker(rank, world, port, q):
    """One rank of tests/test_gpu_tp.py: three consecutive fused exchanges against the oracle."""
    try:
        from oracle import oracle
        pkg = ge.package()
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        torch.cuda.set_device(rank)
        dist.init_process_group("gloo", rank=rank, world_size=world)  # host-side plumbing only
        ctx = pkg.Context(rank, 1 << 20)
        M, K, g = 8, 2560, 256
        handle = ctx.tp_create(rank, world, M, K)
        handles = [None] * world
        dist.all_gather_object(handles, handle)
        ctx.tp_connect(b"".join(handles))
        dist.barrier()
        rng = np.random.default_rng(5)
        x = rng.standard_normal((M, K)).astype(np.float16)
        w = rng.uniform(0.5, 1.5, K).astype(np.float16)
        dx = torch.from_numpy(x).cuda()
        dw = torch.from_numpy(w).cuda()
        ok, msg = True, ""
        for it in range(3):
            parts = [rng.standard_normal((M, K)).astype(np.float16) for _ in range(world)]
            dpart = torch.from_numpy(parts[rank]).cuda()
            dq = torch.empty((M, K), dtype=torch.int8, device="cuda")
            ds = torch.empty((M, K // g), dtype=torch.float32, device="cuda")
            dn = torch.empty((M, K), dtype=torch.float16, device="cuda")
            ctx.tp_allreduce_rmsnorm_quantize(dx, dpart, dw, 1e-6, M, K, g, Xq=dq, Xs=ds, normed_out=dn)
            torch.cuda.synchronize()
            ctx.check_device_status()
            s32 = np.zeros((M, K), np.float32)
            for p_ in parts:                      # ascending rank order, fp32
                s32 = (s32 + p_.astype(np.float32)).astype(np.float32)
            x = oracle.residual_add(x, s32.astype(np.float16))
            if not np.array_equal(dx.cpu().numpy().view(np.uint16), x.view(np.uint16)):
                ok, msg = False, f"iteration {it}: residual stream differs"
                break
            normed = dn.cpu().numpy()
            if oracle.ulp_distance_fp16(normed, oracle.rms_norm(x, w, 1e-6)).max() > 1:
                ok, msg = False, f"iteration {it}: norm off"
                break
            wq, ws = oracle.quantize(normed, g)
            if not (np.array_equal(dq.cpu().numpy(), wq) and np.array_equal(ds.cpu().numpy(), ws)):
                ok, msg = False, f"iteration {it}: codes differ"
                break
        dist.barrier()
        q.put((rank, ok, msg))
        ctx.close()
        dist.destroy_process_group()
    except Exception as e:  # noqa: BLE001
        q.put((rank, False, repr(e)))


def gpu_lm_head_worker(rank, world, port, q):
    """One rank of the column-parallel int8 LM head on GPUs: the packed decode kernel over this rank's rows of a
    [vocab, 2560] head (g256), slices gathered over NCCL. Rows are independent outputs, but the decode kernel's fp32
    summation grouping along K depends on how many row tiles a CTA holds, i.e. on the number of rows in the launch, so
    a shard's logits equal the whole head's only up to fp32 re-association: the bar is the parity bar of the linear
    itself (2 fp16 ulp or 2e-3 relative against the oracle, on 256 sampled rows of the shard), twice that between the
    two launches, with at most max(3, 1e-4 n) elements outside (outputs that are small only because large terms
    cancel; the parity tests count about one per million). What must hold exactly: every rank ends with the same
    gathered bits, and its own slice of them is what it computed."""
    try:
        from oracle import oracle
        from fish_audio_cpp_b200 import lm_head as lmh
        pkg = ge.package()
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        torch.cuda.set_device(rank)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
        ctx = pkg.Context(rank, 1 << 22)
        vocab, K, g = 155776 // 8, 2560, 256  # an eighth of the real head: 19472 rows = 1217 row tiles (odd)
        ok, msg = True, ""

        def outside(a, b, ulp, rel):
            a32, b32 = a.astype(np.float32), b.astype(np.float32)
            good = (oracle.ulp_distance_fp16(a, b) <= ulp) | (np.abs(a32 - b32) <= rel * np.abs(b32))
            return int((~good).sum())

        for M in (1, 8):
            X, W, ws = synth.linear_case(900 + M, M, vocab, K, g)
            dX = torch.from_numpy(X).cuda()
            dW, dS = torch.from_numpy(W).cuda(), torch.from_numpy(ws).cuda()

            def run(Wd, Sd, n):
                packed = torch.empty((ctx.packed_weight_bytes(n, K, g),), dtype=torch.uint8, device="cuda")
                ctx.pack_weight(Wd, Sd, n, K, g, packed)
                ctx.register_packed_weight(Wd, packed, n, K, g)
                Y = torch.empty((M, n), dtype=torch.float16, device="cuda")
                ctx.linear(Wd, Sd, g, dX, Y, M, n, K)
                torch.cuda.synchronize()
                ctx.register_packed_weight(Wd, None)
                return Y

            full = run(dW, dS, vocab)
            lo, hi = lmh.vocab_shard(vocab, world, rank)
            # (a copy of its own, so that the shard is registered under its own address and shape)
            local = run(dW[lo:hi].clone(), dS[lo:hi].clone(), hi - lo)
            got = lmh.gather_logits(torch, dist, local, vocab, world)
            ctx.check_device_status()
            if not torch.equal(got[:, lo:hi].view(torch.int16), local.view(torch.int16)):
                ok, msg = False, f"M={M}: this rank's slice of the gathered logits is not what it computed"
                break
            mine = got.cpu().numpy()
            everyone = [None] * world
            dist.all_gather_object(everyone, mine.view(np.uint16).tobytes())
            if any(e != everyone[0] for e in everyone):
                ok, msg = False, f"M={M}: ranks hold different gathered logits"
                break
            n_out = outside(mine, full.cpu().numpy(), 4, 4e-3)
            if n_out > max(3, int(1e-4 * mine.size)):
                ok, msg = False, f"M={M}: {n_out} of {mine.size} gathered logits are outside the bar against the whole head"
                break
            rows = np.sort(np.random.default_rng(rank).choice(hi - lo, 256, replace=False))
            want = oracle.linear(W[lo:hi][rows], ws[lo:hi][rows], g, X)
            n_out = outside(local.cpu().numpy()[:, rows], want, 2, 2e-3)
            if n_out > 3:
                ok, msg = False, f"M={M}: {n_out} of {want.size} shard logits are outside the bar against the oracle"
                break
        dist.barrier()
        q.put((rank, ok, msg))
        ctx.close()
        dist.destroy_process_group()
    except Exception as e:  # noqa: BLE001
        import traceback
        q.put((rank, False, traceback.format_exc() + repr(e)))


def gpu_stack_worker(rank, world, port, q, tp_mode="fused", layers=2):
    """One rank of the TP-vs-single-GPU test: a `layers`-deep stack of the benchmark's width (hidden 2560, 32 q / 8 kv
    heads, SwiGLU 9728, g256, batch 8, context 1024) cut over `world` ranks runs one decode step; every rank also
    runs the SAME stack uncut on its own GPU and reports how far the tensor-parallel result is from it, next to a
    yardstick: how far the uncut stack's own result moves when every element of its input is moved by one fp16 ulp
    up or down at random. The ranks' outputs are gathered to check that all ranks hold the same bits."""
    try:
        pkg = ge.package()
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        torch.cuda.set_device(rank)
        dist.init_process_group("gloo", rank=rank, world_size=world)  # host-side plumbing only
        B, context = 8, 1024

        def gather(handle):
            out = [None] * world
            dist.all_gather_object(out, handle)
            return out

        report = []
        for n_layer in range(1, layers + 1):
            cfg = S.SlowARConfig(n_layer=n_layer)
            ctx_tp = pkg.Context(rank, 1 << 22)
            st = S.SlowARStack(torch, ctx_tp, cfg, B, context, max_new=8, tp_rank=rank, tp_size=world, seed=31,
                               tp_mode=tp_mode, gather_handles=gather)
            ctx_1 = pkg.Context(rank, 1 << 22)
            solo = S.SlowARStack(torch, ctx_1, cfg, B, context, max_new=8, seed=31)
            rng = np.random.default_rng(23)
            x_np = (rng.standard_normal((B, cfg.dim)) * 0.5).astype(np.float16)
            x_in = torch.from_numpy(x_np).cuda()
            dist.barrier()
            out = st.decode_step(x_in).clone()
            torch.cuda.synchronize()
            ctx_tp.check_device_status()
            want = solo.decode_step(x_in).clone()
            torch.cuda.synchronize()
            jit = (x_np.view(np.uint16).astype(np.int32) + rng.integers(-1, 2, x_np.shape)).astype(np.uint16).view(np.float16)
            solo.reset_positions()
            moved = solo.decode_step(torch.from_numpy(jit).cuda()).clone()
            torch.cuda.synchronize()
            w32 = want.float()
            rel = ((out.float() - w32).norm() / w32.norm()).item()
            noise = ((moved.float() - w32).norm() / w32.norm()).item()
            ulp = (out.view(torch.int16).int() - want.view(torch.int16).int()).abs()
            same = (ulp == 0).float().mean().item()
            bits = out.cpu().numpy().view(np.uint16).copy()
            all_bits = [None] * world
            dist.all_gather_object(all_bits, bits)
            identical = all(np.array_equal(all_bits[0], b) for b in all_bits)
            report.append(dict(layers=n_layer, rel=rel, noise=noise, same_bits=same, ranks_identical=identical))
            st.close(); solo.close()
            ctx_tp.close(); ctx_1.close()
            del st, solo
            torch.cuda.empty_cache()
        dist.barrier()
        q.put((rank, True, report))
        dist.destroy_process_group()
    except Exception as e:  # noqa: BLE001
        import traceback
        q.put((rank, False, traceback.format_exc() + repr(e)))
