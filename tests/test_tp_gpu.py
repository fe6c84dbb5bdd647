"""Tensor-parallel Int8 OPT on real GPUs (NCCL): the logits of a tp=2 (and tp=4) run must be
bit-identical to the single-GPU run of the same model, because only int32 partial sums are
exchanged.  Needs at least 2 GPUs; skipped otherwise.  The fused attention kernel and the three-kernel
chain are deterministic per row, so the comparison holds with either."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, ret, big):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    import datetime
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank),
                            timeout=datetime.timedelta(seconds=120))
    try:
        from torch_int import _CUDA as C
        from torch_int.models.opt import Int8OPTConfig
        from torch_int.models.random_init import random_int8_opt
        from torch_int.models.tensor_parallel import TensorParallel
        if big:
            # two layers at the OPT-175B dimensions: the per-rank GEMM, attention and exchange shapes of the
            # tensor-parallel benchmark (prefill groups of 1024 tokens, decode steps of 8 rows)
            cfg = Int8OPTConfig(vocab_size=512, hidden_size=12288, num_hidden_layers=2, ffn_dim=49152,
                                num_attention_heads=96, max_position_embeddings=640)
            shapes, shapes4, prompt, new = (1, 520), (8, 512), 24, 4
        else:
            cfg = Int8OPTConfig(vocab_size=512, hidden_size=512, num_hidden_layers=3, ffn_dim=2048,
                                num_attention_heads=8, max_position_embeddings=256)
            shapes, shapes4, prompt, new = (2, 77), (4, 48), 20, 5
        dev = torch.device("cuda", rank)
        tp_model = random_int8_opt(cfg, seed=21, device=dev, tp=TensorParallel.from_world(), consistent=True)
        if not big:
            tp_model.model.decoder.tp.min_pipeline_tokens = 32  # exercise the pipelined loop at test sizes
        g = torch.Generator().manual_seed(5)
        ids = torch.randint(0, cfg.vocab_size, shapes, generator=g).to(dev)
        logits = tp_model(ids).logits                       # one group of sequences
        ids4 = torch.randint(0, cfg.vocab_size, shapes4, generator=g).to(dev)
        logits4 = tp_model(ids4).logits                     # several groups: pipelined exchanges
        again = tp_model(ids4).logits                       # a second pass over the same workspace
        gen = tp_model.generate_greedy(ids4[:, :prompt], new)   # static cache, one-token steps
        if not big:
            # the default replays the steps from a CUDA graph that contains the NCCL all-reduces: same tokens
            # as eager steps
            assert tp_model.model.decoder.tp.decode_graph
            eager = tp_model.generate_greedy(ids4[:, :prompt], new, use_cuda_graph=False)
            if not torch.equal(gen, eager):
                raise AssertionError("graph replay of tensor-parallel decode steps differs from eager steps")
        tp = tp_model.model.decoder.tp
        extra_ok = True
        if not big:
            # checkpoint round trip under tensor parallelism: rank 0 writes the whole model, every rank
            # reads only its slices of it, and the logits stay bit-identical
            import tempfile
            from torch_int.models.opt import Int8OPTForCausalLM
            box = [tempfile.mkdtemp(prefix="ti_ckpt_") if rank == 0 else None]
            dist.broadcast_object_list(box, src=0)
            if rank == 0:
                random_int8_opt(cfg, seed=21, device=dev, tp=TensorParallel.single(), consistent=True).save_pretrained(box[0])
            dist.barrier()
            loaded = Int8OPTForCausalLM.from_pretrained(box[0], device=dev, tp=TensorParallel.from_world())
            loaded.model.decoder.tp.min_pipeline_tokens = 32
            extra_ok = extra_ok and torch.equal(loaded(ids4).logits, logits4)
            # vocabulary-parallel language-model head: each rank multiplies with its rows of the tied table
            vp = loaded.model.decoder.tp
            vp.vocab_parallel = True
            split = loaded(ids4).logits
            vp.vocab_parallel = False
            scale = float(logits4.abs().max())
            extra_ok = extra_ok and split.shape == logits4.shape and float((split - logits4).abs().max()) <= 1e-4 * scale
            extra_ok = extra_ok and torch.equal(split.argmax(-1), logits4.argmax(-1))
            del loaded
            dist.barrier()
            if rank == 0:
                import shutil
                shutil.rmtree(box[0], ignore_errors=True)
        peer = tp.use_peer_memory and len(tp._workspaces) > 0  # the fused peer-memory exchange really ran
        checked = all(ws.checked for ws in tp._workspaces.values())
        status = C.device_status()
        del tp_model
        torch.cuda.empty_cache()
        ok = True
        if rank == 0:
            one = random_int8_opt(cfg, seed=21, device=dev, tp=TensorParallel.single(), consistent=True)
            ok = (torch.equal(logits, one(ids).logits) and torch.equal(logits4, one(ids4).logits)
                  and torch.equal(again, logits4) and torch.equal(gen, one.generate_greedy(ids4[:, :prompt], new)))
        ret[rank] = (bool(ok and peer and checked and extra_ok), status)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,big", [(2, False), (4, False), (4, True)])
def test_tp_logits_equal_single_gpu(world, big):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=_rank_main, args=(r, world, port, ret, big)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=420)
        assert p.exitcode == 0, f"rank exited with {p.exitcode}"
    for r in range(world):
        ok, status = ret[r]
        assert ok and status == 0, f"rank {r}: equal={ok} status={status}"
