"""N-column sharding: the partition rule and the gathered layout, with world_size-2 gloo ranks on CPU; the
multi-device path on GPUs when more than one is present."""
import os
import socket
import subprocess
import sys
import textwrap

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_shard_columns_rule(t0):
    assert t0.shard_columns(16384, 8, 0) == (0, 2048)
    assert t0.shard_columns(16384, 8, 7) == (14336, 2048)
    assert t0.shard_columns(4096, 1, 0) == (0, 4096)
    covered = []
    for r in range(4):
        first, cnt = t0.shard_columns(1024, 4, r)
        covered += list(range(first, first + cnt))
    assert covered == list(range(1024))
    with pytest.raises(t0.T0Error):
        t0.shard_columns(1000, 3, 0)       # ragged N is refused
    with pytest.raises(t0.T0Error):
        t0.shard_columns(1024, 4, 4)


_WORKER = textwrap.dedent("""
    import importlib, os, sys
    import numpy as np, torch, torch.distributed as dist
    sys.path.insert(0, {root!r})
    t0 = importlib.import_module("rust-gpu_b200")
    import oracle
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    M, N, K = 24, 64, 96
    a = oracle.fill_uniform_bf16(M * K, 42 + M)                       # A is replicated: every rank regenerates it
    first, cnt = t0.shard_columns(N, world, rank)
    # rank r owns rows [first, first+cnt) of WT[N,K]: the same stream, offset by its first element (as bench.py does)
    b_slice = oracle.fill_uniform_bf16(cnt * K, 137 + N, first * K)
    y_slice = oracle.gemm_nt(a, b_slice, M, K, cnt)                   # stand-in for the rank's GPU kernel on CPU ranks
    blocks = [torch.empty(M, cnt) for _ in range(world)]              # rank-major C_g[g][M][N/g]
    dist.all_gather(blocks, torch.from_numpy(y_slice))
    gathered = torch.stack(blocks)
    full = oracle.gemm_nt(a, oracle.fill_uniform_bf16(N * K, 137 + N), M, K, N)
    rebuilt = np.concatenate([gathered[r].numpy() for r in range(world)], axis=1)
    assert np.array_equal(rebuilt, full), "gathered blocks do not reassemble to the full product"
    # timing rule of the benchmark: the reported time is the max over ranks
    t = torch.tensor([1.0 + rank], dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    assert t.item() == float(world)
    dist.destroy_process_group()
    print("rank", rank, "ok")
""")


def test_two_rank_gloo_sharded_gemm_and_gather(t0, oracle, tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(_WORKER.format(root=ROOT))
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    procs = []
    for rank in range(2):
        env = dict(os.environ, RANK=str(rank), WORLD_SIZE="2", MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), LOCAL_RANK=str(rank))
        procs.append(subprocess.Popen([sys.executable, str(script)], env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    outs = [p.communicate(timeout=300)[0] for p in procs]
    for rank, (p, out) in enumerate(zip(procs, outs)):
        assert p.returncode == 0, out
        assert f"rank {rank} ok" in out


def test_bench_reference_arm_other_ranks_exit_quietly():
    # under torchrun only rank 0 runs the CPU reference arm; the other ranks exit 0 without output
    env = dict(os.environ, RANK="1", WORLD_SIZE="2", LOCAL_RANK="1")
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "2", "--steps", "1", "--warmup", "0"],
                       env=env, capture_output=True, text=True, timeout=120)
    assert r.returncode == 0 and r.stdout.strip() == ""


@pytest.mark.gpu
def test_multi_device_sharded_gemm_and_gather(t0, oracle):
    import torch
    g = min(torch.cuda.device_count(), 4)
    if g < 2:
        pytest.skip("needs at least two GPUs")       # like the reference's multi-GPU tests (src/universal/multi_gpu_tests.rs:64-70)
    M, N, K = 256, 512 * g, 256
    mg = t0.MultiGpu(g)
    a = oracle.fill_uniform_bf16(M * K, 42 + M)
    b = oracle.fill_uniform_bf16(N * K, 137 + N)
    xs, bs, cs = [], [], []
    for r in range(g):
        rt = mg.runtime(r)
        first, cnt = t0.shard_columns(N, g, r)
        xs.append(rt.upload(a)); bs.append(rt.upload(b.reshape(N, K)[first:first + cnt])); cs.append(rt.alloc_zero(M * N * 4))
    cnt = N // g
    mg.gemm_sharded([x.gpu_addr() for x in xs], [x.gpu_addr() for x in bs], [c.gpu_addr() + r * M * cnt * 4 for r, c in enumerate(cs)], M, N, K)
    mg.all_gather_c([c.gpu_addr() for c in cs], M, N)
    mg.synchronize()
    full = oracle.gemm_nt(a, b, M, K, N)
    for r in range(g):
        blocks = cs[r].read(M * N * 4, np.float32).reshape(g, M, cnt)
        rebuilt = np.concatenate(list(blocks), axis=1)
        assert np.abs(rebuilt - full).max() <= 5e-3 and np.linalg.norm(rebuilt - full) / np.linalg.norm(full) <= 1e-3
    mg.free()


@pytest.mark.gpu
def test_gather_launch_with_extra_destinations_on_one_gpu(t0, oracle):
    # the gathered-output launch writes the same product to args.y and to every further destination; on one GPU the further
    # destinations are ordinary buffers of the same device.  Several tiles per CTA, ragged M (the copies clip rows >= M),
    # both kernels, and the shapes the entry must refuse.
    rt = t0.GpuRuntime(0)
    try:
        for (M, N, K, pair) in [(300, 512, 256, 2), (1000, 1024, 128, 1), (4096 + 40, 2048, 64, 1)]:
            a = oracle.fill_uniform_bf16(M * K, 1 + M)
            b = oracle.fill_uniform_bf16(N * K, 2 + N)
            xa, xb = rt.upload(a), rt.upload(b)
            dests = [rt.alloc(M * N * 4 + 4096) for _ in range(4)]
            for d in dests:
                d.write(np.full(M * N + 1024, -777.0, np.float32))
            args = rt.gemm_args(xa.gpu_addr(), xb.gpu_addr(), dests[0].gpu_addr(), M, N, K, pair_cta=pair)
            rt.gemm_gather(args, [d.gpu_addr() for d in dests[1:]])
            rt.synchronize()
            ref = oracle.gemm_nt(a, b, M, K, N)
            first = dests[0].read((M * N + 1024) * 4, np.float32)
            assert np.abs(first[:M * N].reshape(M, N) - ref).max() <= 5e-3 * np.sqrt(max(K, 256) / 256)
            assert np.all(first[M * N:] == -777.0), "wrote past the matrix"
            for d in dests[1:]:
                assert np.array_equal(d.read((M * N + 1024) * 4, np.float32), first)
            for buf in [xa, xb] + dests:
                buf.free()
        xa, xb, y = rt.alloc(64 * 64 * 2), rt.alloc(80 * 64 * 2), rt.alloc(64 * 80 * 4)
        with pytest.raises(t0.T0Error):          # N % 32 != 0: some chunks would not go through the TMA store
            rt.gemm_gather(rt.gemm_args(xa.gpu_addr(), xb.gpu_addr(), y.gpu_addr(), 64, 80, 64), [y.gpu_addr()])
        with pytest.raises(t0.T0Error):          # split-K
            rt.gemm_gather(rt.gemm_args(xa.gpu_addr(), xb.gpu_addr(), y.gpu_addr(), 64, 64, 64, split_k=2), [y.gpu_addr()])
    finally:
        rt.close()


@pytest.mark.gpu
def test_multi_device_gemm_with_gather_in_the_epilogue(t0, oracle):
    # GEMM and all-gather in one kernel per GPU: afterwards every GPU holds all of C in C_g[g][M][N/g], equal bit for bit to
    # what the GEMM + NCCL all-gather pair leaves
    import torch
    g = min(torch.cuda.device_count(), 4)
    if g < 2:
        pytest.skip("needs at least two GPUs")
    M, N, K = 1000, 512 * g, 512
    mg = t0.MultiGpu(g)
    a = oracle.fill_uniform_bf16(M * K, 42 + M)
    b = oracle.fill_uniform_bf16(N * K, 137 + N)
    cnt = N // g
    xs, bs, cs, cn = [], [], [], []
    for r in range(g):
        rt = mg.runtime(r)
        xs.append(rt.upload(a)); bs.append(rt.upload(b.reshape(N, K)[r * cnt:(r + 1) * cnt]))
        cs.append(rt.alloc_zero(M * N * 4)); cn.append(rt.alloc_zero(M * N * 4))
    mg.gemm_sharded_gathered([x.gpu_addr() for x in xs], [x.gpu_addr() for x in bs], [c.gpu_addr() for c in cs], M, N, K)
    mg.synchronize()
    mg.gemm_sharded([x.gpu_addr() for x in xs], [x.gpu_addr() for x in bs], [c.gpu_addr() + r * M * cnt * 4 for r, c in enumerate(cn)], M, N, K,
                    tile_n=256)
    mg.all_gather_c([c.gpu_addr() for c in cn], M, N)
    mg.synchronize()
    full = oracle.gemm_nt(a, b, M, K, N)
    for r in range(g):
        got = cs[r].read(M * N * 4, np.float32)
        rebuilt = np.concatenate(list(got.reshape(g, M, cnt)), axis=1)
        assert np.abs(rebuilt - full).max() <= 5e-3 * np.sqrt(K / 256)
        assert np.array_equal(got, cn[r].read(M * N * 4, np.float32)), f"GPU {r}: one-kernel gather differs from GEMM + all-gather"
    mg.free()


@pytest.mark.gpu
def test_multi_device_host_operands_upload_a_once(t0, oracle):
    # host operands: every GPU uploads 1/g of A, the GPUs complete their copies over NVLink, each returns its column block
    # of C into the caller's row-major matrix; ragged M (rows not a multiple of g) included
    import torch
    g = min(torch.cuda.device_count(), 4)
    if g < 2:
        pytest.skip("needs at least two GPUs")
    mg = t0.MultiGpu(g)
    for (M, N, K) in [(1000, 256 * g, 512), (4096, 1024 * g, 1024)]:
        a = oracle.fill_uniform_bf16(M * K, 42 + M)
        b = oracle.fill_uniform_bf16(N * K, 137 + N)
        y = np.full(M * N, -9999.0, np.float32)
        for _ in range(2):                      # the second call reuses the handle's device buffers
            y[:] = -9999.0
            mg.gemm_sharded_host(a, b, y, M, N, K)
            full = oracle.gemm_nt(a, b, M, K, N)
            got = y.reshape(M, N)
            assert np.abs(got - full).max() <= 5e-3 * np.sqrt(K / 256) and np.linalg.norm(got - full) / np.linalg.norm(full) <= 1e-3
    mg.free()


@pytest.mark.gpu
def test_sharded_16384_every_rank_checked(t0, oracle):
    # the sharded configuration at full size: GPU r computes the 16384 x (16384/g) x 16384 block of its rows of WT (the same
    # seeded stream, offset by the block's first element); 64 rows spread over the whole matrix are compared on EVERY rank
    import torch
    g = min(torch.cuda.device_count(), 8)
    if g < 2:
        pytest.skip("needs at least two GPUs")
    M = N = K = 16384
    n_local = N // g
    mg = t0.MultiGpu(g)
    xs, bs, cs = [], [], []
    for r in range(g):
        rt = mg.runtime(r)
        first, cnt = t0.shard_columns(N, g, r)
        assert (first, cnt) == (r * n_local, n_local)
        xa, xb, y = rt.alloc(M * K * 2), rt.alloc(cnt * K * 2), rt.alloc(M * cnt * 4)
        rt.fill_uniform_bf16(xa.gpu_addr(), M * K, 42 + M)
        rt.fill_uniform_bf16(xb.gpu_addr(), cnt * K, 137 + N, first * K)
        xs.append(xa); bs.append(xb); cs.append(y)
    mg.gemm_sharded([x.gpu_addr() for x in xs], [x.gpu_addr() for x in bs], [c.gpu_addr() for c in cs], M, N, K)
    mg.synchronize()
    rows = [(i * 257 + 13) % M for i in range(64)]
    a_rows = np.concatenate([oracle.fill_uniform_bf16(K, 42 + M, r * K) for r in rows])
    for r in range(g):
        b_slice = oracle.fill_uniform_bf16(n_local * K, 137 + N, r * n_local * K)
        ref = oracle.gemm_nt(a_rows, b_slice, len(rows), K, n_local)
        got = np.stack([cs[r].read_bytes(row * n_local * 4, n_local * 4, np.float32) for row in rows])
        assert np.abs(got - ref).max() <= 5e-3 * np.sqrt(K / 256), f"rank {r}"
        assert np.linalg.norm(got - ref) / np.linalg.norm(ref) <= 1e-3, f"rank {r}"
    for b in xs + bs + cs:
        b.free()
    mg.free()
