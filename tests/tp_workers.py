"""Worker functions for the two-rank tensor-parallel tests (spawned with torch.multiprocessing)."""
import os
import sys
from pathlib import Path

import numpy as np
import torch
import torch.distributed as dist

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def _cfg(kind="llama"):
    from oracle import token_loop_oracle as O

    if kind == "moe_tp":
        # Qwen3-MoE wiring with the reference's own tensor-parallel layout: every rank holds a slice of
        # every expert's intermediate dimension (src/moe/moe.cc:22-30), 2 kv heads split over the ranks
        return O.ModelConfig(2, 256, 4, 2, 128, 512, 1024, 1e-6, 1e6, 256, False, True, True, "silu",
                             8, 2, 256, True)
    if kind == "moe_ep":
        # Qwen3-MoE wiring, 8 experts top-2 partitioned over the ranks, and ONE kv head for 4 q heads
        # so that the kv head is replicated on both ranks (the shape of the 30B-A3B config at 8 GPUs)
        return O.ModelConfig(2, 256, 4, 1, 128, 512, 1024, 1e-6, 1e6, 256, False, True, True, "silu",
                             8, 2, 128, True)
    # Llama wiring (the TP benchmark architecture), 2 layers, 4 q / 2 kv heads so that 2 ranks divide them
    return O.ModelConfig(2, 256, 4, 2, 128, 512, 1024, 1e-5, 5e5, 256, False, False, False)


def _batch(cfg, prompts):
    from oracle import token_loop_oracle as O

    ids, pos, loc, qo, cur = [], [], [], [0], 0
    pt = np.zeros((len(prompts), 64), dtype=np.int32)
    for b, p in enumerate(prompts):
        for i, t in enumerate(p):
            ids.append(t)
            pos.append(i)
            loc.append(cur)
            pt[b, i] = cur
            cur += 1
        qo.append(len(ids))
    return O.StepBatch(np.array(ids, np.int32), np.array(pos, np.int32), np.array(loc, np.int32),
                       np.arange(len(prompts), dtype=np.int32), np.array([len(p) for p in prompts], np.int32),
                       np.array(qo, np.int32), True), pt, cur


def cpu_oracle_worker(rank, world, port, out_path, kind="llama"):
    """Each gloo rank runs the oracle on its weight shard with dist.all_reduce where the reference
    all-reduces; rank 0 saves the logits for comparison with the unsharded oracle."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import __graft_entry__ as entry
    from oracle import token_loop_oracle as O

    entry.load_package()
    from sglang_cpp_b200 import tp

    cfg = _cfg(kind)
    ep = kind == "moe_ep"
    w = O.init_weights(cfg, seed=0, std=0.05, router_std=1.0 if kind.startswith("moe") else None)
    rng = np.random.default_rng(0)
    prompts = [rng.integers(0, cfg.vocab_size, size=n).tolist() for n in (7, 19)]
    batch, pt, slots = _batch(cfg, prompts)

    def all_reduce(t):
        t = t.clone()
        dist.all_reduce(t)
        return t

    lcfg = tp.local_config(cfg, world, ep)
    local = O.OracleModel(lcfg, tp.shard_weights(cfg, w, rank, world, ep), O.store_fp32, all_reduce,
                          expert_begin=rank * cfg.num_experts // world if ep else 0)
    kv = O.KVState.create(lcfg, slots + 1)
    logits = local.forward(batch, kv, pt)
    if rank == 0:
        full = O.OracleModel(cfg, w, O.store_fp32)
        want = full.forward(batch, O.KVState.create(cfg, slots + 1), pt)
        torch.save({"got": logits, "want": want}, out_path)
    dist.barrier()
    dist.destroy_process_group()


def _init_group(rank, world, port, symmetric):
    """gloo for the host-side exchanges; with `symmetric` also NCCL, whose group torch's symmetric-memory
    rendezvous (peer and multicast addresses of the exchange buffers) runs on."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    if symmetric:
        dist.init_process_group("cpu:gloo,cuda:nccl", rank=rank, world_size=world,
                                device_id=torch.device("cuda", rank))
    else:
        dist.init_process_group("gloo", rank=rank, world_size=world)


def gpu_engine_worker(rank, world, port, out_path, kind="llama", symmetric=False):
    """Two processes, one GPU each: the engine with tp_size = 2 (fused all-reduce over peer memory)
    against the unsharded oracle, prefill then decode.  symmetric: the exchange buffers are a
    symmetric-memory allocation and the all-reduce is summed in the NVLink switch."""
    _init_group(rank, world, port, symmetric)
    import __graft_entry__ as entry
    from oracle import token_loop_oracle as O

    pkg = entry.load_package()
    pkg.load_library()
    from sglang_cpp_b200.engine import Engine, EngineConfig
    from sglang_cpp_b200.host_batch import HostBatcher

    cfg = _cfg(kind)
    ep = kind == "moe_ep"
    w = O.init_weights(cfg, seed=0, std=0.02, router_std=1.0 if kind.startswith("moe") else None)
    eng = Engine(cfg, EngineConfig(16, 32, 4, 256, 512, rank, world, ep))
    eng.load_weights(w, rank, world)
    eng.connect_tp(symmetric=symmetric)
    if symmetric and rank == 0:
        from sglang_cpp_b200._lib import load as _load_lib
        import ctypes as _ct
        _load_lib().b200_engine_comm.restype = _ct.c_void_p
        res_multicast = bool(_load_lib().b200_comm_uses_multicast(_ct.c_void_p(_load_lib().b200_engine_comm(eng._h))))
    hb = HostBatcher(eng, 32, 16, 4, enable_prefix_cache=False)
    rng = np.random.default_rng(0)
    prompts = [rng.integers(0, cfg.vocab_size, size=n).astype(np.int32) for n in (7, 19)]
    reqs = [hb.add_request(p, 8) for p in prompts]
    out = hb.prefill(reqs)
    out.synchronize()
    res = {"prefill": eng.logits(2).clone()}
    if symmetric and rank == 0:
        res["multicast"] = res_multicast
    toks = [out.next_tokens_cpu.clone()]
    decode_logits = []
    for _ in range(3):
        out = hb.decode(reqs)
        out.synchronize()
        toks.append(out.next_tokens_cpu.clone())
        decode_logits.append(eng.logits(2).clone())
    res["decode_logits"] = torch.stack(decode_logits)
    res["tokens"] = torch.stack(toks)
    # both ranks must agree bit for bit (same sums in the same rank order)
    gathered = [None] * world
    dist.all_gather_object(gathered, (res["decode_logits"], res["tokens"]))
    if rank == 0:
        res["ranks_agree"] = all(torch.equal(g[0], gathered[0][0]) and torch.equal(g[1], gathered[0][1]) for g in gathered)
        # the oracle, unsharded, on the same requests; decode steps are fed the engine's own tokens
        model = O.OracleModel(cfg, w, O.store_bf16)
        kv = O.KVState.create(cfg, 33 * 16)
        pt = np.zeros((5, 256), dtype=np.int32)
        for r in reqs:
            pt[r.table_idx] = hb.slots_of(r)[:256]
        ids, pos, loc, qo = [], [], [], [0]
        for r, p in zip(reqs, prompts):
            for i, t in enumerate(p):
                ids.append(int(t)); pos.append(i); loc.append(int(pt[r.table_idx, i]))
            qo.append(len(ids))
        rows = np.array([r.table_idx for r in reqs], np.int32)
        b = O.StepBatch(np.array(ids, np.int32), np.array(pos, np.int32), np.array(loc, np.int32), rows,
                        np.array([len(p) for p in prompts], np.int32), np.array(qo, np.int32), True)
        res["want_prefill"] = model.forward(b, kv, pt)
        want_decode = []
        for k in range(3):
            at = np.array([len(p) + k for p in prompts], np.int32)
            b = O.StepBatch(res["tokens"][k].numpy().astype(np.int32), at,
                            np.array([pt[r.table_idx, a] for r, a in zip(reqs, at)], np.int32), rows,
                            at + 1, np.arange(3, dtype=np.int32), False)
            want_decode.append(model.forward(b, kv, pt))
        res["want_decode"] = torch.stack(want_decode)
        torch.save(res, out_path)
    dist.barrier()
    eng.close()
    dist.destroy_process_group()


def gpu_allreduce_worker(rank, world, port, out_path, stress_calls=0, symmetric=False):
    """The all-reduce calls of the C ABI on their own (tensor_model_parallel_all_reduce and its
    fusion with add + norm), several calls in a row so that both buffer parities and the call
    numbering are exercised; rank 0 saves what it got and what the sums should be."""
    _init_group(rank, world, port, symmetric)
    import ctypes
    import __graft_entry__ as entry
    from oracle import token_loop_oracle as O

    pkg = entry.load_package()
    lib = pkg.load_library()
    from sglang_cpp_b200._lib import call
    from sglang_cpp_b200.tp import exchange_handles

    rows, hidden = 37, 1024
    comm = ctypes.c_void_p()
    if symmetric:
        import torch.distributed._symmetric_memory as symm_mem

        nbytes = int(lib.b200_comm_region_bytes(rows * hidden * 2))
        region = symm_mem.empty(nbytes, dtype=torch.uint8, device=torch.device("cuda", rank))
        region.zero_()
        torch.cuda.synchronize()
        handle = symm_mem.rendezvous(region, dist.group.WORLD.group_name)
        call("b200_comm_create_on", rank, world, rows * hidden * 2, region.data_ptr(), ctypes.byref(comm))
        peers = (ctypes.c_void_p * world)(*[int(p) for p in handle.buffer_ptrs])
        call("b200_comm_connect_pointers", comm, peers, int(handle.multicast_ptr) if handle.multicast_ptr else None)
        dist.barrier()
    else:
        call("b200_comm_create", rank, world, rows * hidden * 2, ctypes.byref(comm))
        n = lib.b200_comm_handle_bytes()
        buf = ctypes.create_string_buffer(n)
        call("b200_comm_export", comm, buf)
        call("b200_comm_connect", comm, exchange_handles(buf.raw, rank, world))
    gen = torch.Generator().manual_seed(17)
    res = {"plain": [], "want_plain": [], "fused_x": [], "fused_res": [], "want_x": [], "want_res": []}
    weight = (torch.randn(hidden, generator=gen) * 0.1 + 1).to(torch.bfloat16)
    residual0 = (torch.randn(rows, hidden, generator=gen)).to(torch.bfloat16)
    residual = residual0.cuda()
    want_res = residual0.clone()
    stream = torch.cuda.current_stream().cuda_stream
    for c in range(5):
        parts = [(torch.randn(rows, hidden, generator=gen)).to(torch.bfloat16) for _ in range(world)]
        total = sum(p.float() for p in parts).to(torch.bfloat16)        # fp32 sum in rank order, one rounding
        ptr = lib.b200_comm_buffer(comm, c & 1)
        from sglang_cpp_b200.engine import _as_cuda_tensor
        _as_cuda_tensor(ptr, rows * hidden * 2).view(torch.bfloat16).copy_(parts[rank].cuda().flatten())
        torch.cuda.synchronize()
        out = torch.empty(rows, hidden, dtype=torch.bfloat16, device="cuda")
        if c % 2 == 0:
            call("b200_allreduce", comm, c & 1, out.data_ptr(), rows, hidden, stream)
            torch.cuda.synchronize()
            res["plain"].append(out.cpu())
            res["want_plain"].append(total)
        else:
            call("b200_allreduce_fused_add_rmsnorm", comm, c & 1, out.data_ptr(), residual.data_ptr(),
                 weight.cuda().data_ptr(), rows, hidden, 1e-6, 1, stream)
            torch.cuda.synchronize()
            want_res = (total.float() + want_res.float()).to(torch.bfloat16)
            res["fused_x"].append(out.cpu())
            res["fused_res"].append(residual.cpu().clone())
            res["want_x"].append(O.rmsnorm(want_res, weight, 1e-6))
            res["want_res"].append(want_res.clone())
        dist.barrier()
    # Long run with no host synchronisation between calls: each rank fills its exchange buffer on the
    # device and calls again at once, alternating the plain and the fused form and the buffer parity,
    # so a rank runs ahead of its peer whenever the protocol lets it.  Every sum is checked on the
    # device against the same fp32-in-rank-order sum computed locally; mismatching calls are counted.
    bad = torch.zeros(1, dtype=torch.int64, device="cuda")

    def differs(got, want, summed=None):
        # peer-memory kernels: the fp32 sum in rank order rounded once, bit for bit.  In-switch sums
        # (symmetric): the switch's own rounding of the sum, within one bf16 step of that sum (and,
        # in the fused form, one more step of the residual it is added to).
        if not symmetric:
            return got != want
        step = want.float().abs() * 2 ** -7 + 1e-6
        if summed is not None:
            step = step + summed.float().abs() * 2 ** -7
        return (got.float() - want.float()).abs() > step

    from sglang_cpp_b200.engine import _as_cuda_tensor
    bufs = [_as_cuda_tensor(lib.b200_comm_buffer(comm, par), rows * hidden * 2).view(torch.bfloat16).view(rows, hidden)
            for par in (0, 1)]
    w_dev = weight.cuda()
    out = torch.empty(rows, hidden, dtype=torch.bfloat16, device="cuda")
    g = torch.Generator(device="cuda")
    for c in range(5, 5 + stress_calls):
        parts = []
        for r in range(world):
            g.manual_seed(1000 * c + r)
            parts.append(torch.randn(rows, hidden, generator=g, device="cuda").to(torch.bfloat16))
        total = sum(p.float() for p in parts).to(torch.bfloat16)
        bufs[c & 1].copy_(parts[rank])
        if c % 2 == 0:
            call("b200_allreduce", comm, c & 1, out.data_ptr(), rows, hidden, stream)
            bad += differs(out, total).any().long()
        else:
            before = residual.clone()
            call("b200_allreduce_fused_add_rmsnorm", comm, c & 1, out.data_ptr(), residual.data_ptr(),
                 w_dev.data_ptr(), rows, hidden, 1e-6, 1, stream)
            bad += differs(residual, (total.float() + before.float()).to(torch.bfloat16), total).any().long()
            residual.mul_(0.5)   # keep the running residual bounded
    torch.cuda.synchronize()
    res["stress_calls"] = stress_calls
    res["stress_bad"] = int(bad.item())
    res["multicast"] = bool(lib.b200_comm_uses_multicast(comm))
    allbad = [None] * world
    dist.all_gather_object(allbad, res["stress_bad"])
    res["stress_bad_all_ranks"] = allbad
    if rank == 0:
        torch.save(res, out_path)
    dist.barrier()
    call("b200_comm_destroy", comm)
    dist.destroy_process_group()
