"""Tensor-parallel host logic on CPU ranks (gloo, world size 2 and 4): the weight
sharder and the int32 all-reduce wrapper of the product, with the per-rank
arithmetic done by the oracle.  The sharded evaluation must equal the unsharded
oracle bit for bit, because the exchanged partial sums are integers."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import opt_model as OM
from oracle import w8a8 as O


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _model_sd(hidden=128, heads=4, ffn=256, layers=1, seed=3):
    from torch_int.models.opt import Int8OPTConfig
    from torch_int.models.random_init import random_int8_opt
    cfg = Int8OPTConfig(vocab_size=64, hidden_size=hidden, num_hidden_layers=layers, ffn_dim=ffn,
                        num_attention_heads=heads, max_position_embeddings=64)
    model = random_int8_opt(cfg, seed=seed, device="cpu")
    return cfg, {k: v.detach() for k, v in model.state_dict().items()}


def _rank_main(rank, world, port, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from torch_int.models.tensor_parallel import TensorParallel
        torch.set_num_threads(1)
        tp = TensorParallel.from_world()
        assert (tp.size, tp.rank) == (world, rank)
        cfg, full = _model_sd()
        sd = tp.shard_state_dict(full)
        e, heads = cfg.hidden_size, cfg.num_attention_heads
        hl, d = heads // world, e // heads
        p = "model.decoder.layers.0"
        assert sd[p + ".self_attn.q_proj.weight"].shape == (e // world, e)
        assert sd[p + ".self_attn.q_proj.bias"].shape == (1, e // world)
        assert sd[p + ".self_attn.out_proj.weight"].shape == (e, e // world)
        assert sd[p + ".self_attn.out_proj.bias"].shape == (1, e)
        assert sd[p + ".fc1.weight"].shape == (cfg.ffn_dim // world, e)
        assert sd[p + ".fc2.weight"].shape == (e, cfg.ffn_dim // world)
        g = torch.Generator().manual_seed(11)
        hidden = torch.randn((2, 16, e), generator=g)
        mask = O.causal_mask(2, 16, 16)
        bsz, tgt = 2, 16
        # --- this rank's part of the layer, with the product's all-reduce in the two exchange steps
        residual = hidden.clone()
        h8 = O.layernorm_q(residual, sd[p + ".self_attn_layer_norm.weight"], sd[p + ".self_attn_layer_norm.bias"], 1e-5)
        x2d = h8.view(-1, e)

        def shape(t):
            return t.view(bsz, tgt, hl, d).transpose(1, 2).reshape(bsz * hl, tgt, d).contiguous()

        a = p + ".self_attn"
        q, k, v = (shape(OM._linear_s8(sd, f"{a}.{n}", x2d)) for n in ("q_proj", "k_proj", "v_proj"))
        probs = O.softmax_q(O.bmm_s8t_s8n_f32t(q, k, float(sd[a + ".qk_bmm.a"])), mask)
        ctx = O.bmm_s8t_s8n_s8t(probs, v.transpose(1, 2).contiguous(), float(sd[a + ".pv_bmm.a"]))
        ctx = ctx.view(bsz, hl, tgt, d).transpose(1, 2).reshape(bsz * tgt, hl * d).contiguous()
        part = tp.all_reduce_int32(OM.row_parallel_partial(ctx, sd[a + ".out_proj.weight"]))
        residual, h8 = O.dq_add_layernorm_q_bias(part.view(bsz, tgt, e), float(sd[a + ".out_proj.a"]),
                                                 sd[a + ".out_proj.bias"].reshape(-1), residual,
                                                 sd[p + ".final_layer_norm.weight"], sd[p + ".final_layer_norm.bias"], 1e-5)
        f8 = OM._linear_s8(sd, p + ".fc1", h8.view(-1, e), relu=True)
        part = tp.all_reduce_int32(OM.row_parallel_partial(f8, sd[p + ".fc2.weight"]))
        residual, _ = O.dq_add_layernorm_q_bias(part.view(bsz, tgt, e), float(sd[p + ".fc2.a"]),
                                                sd[p + ".fc2.bias"].reshape(-1), residual,
                                                torch.ones(e), torch.zeros(e), 1e-5)
        want, _ = OM.decoder_layer(full, p, hidden, mask, heads)
        ok = torch.equal(residual, want)
        # a float tensor must be refused: the exchange is defined on int32 partial sums only
        refused = False
        try:
            tp.all_reduce_int32(torch.zeros(4))
        except RuntimeError:
            refused = True
        # vocabulary-parallel language-model head: every rank multiplies with its rows of the tied
        # embedding table; the gathered logits equal the whole product (same dot products, fp32)
        table = full["model.decoder.embed_tokens.weight"]
        whole = torch.nn.functional.linear(residual, table)
        split = tp.vocab_parallel_logits(residual, table)
        ok = ok and split.shape == whole.shape and torch.allclose(split, whole, rtol=1e-5, atol=1e-5)
        odd = torch.randn((world * 3 + 1, e), generator=g)       # a vocabulary that does not divide: whole product
        ok = ok and torch.equal(tp.vocab_parallel_logits(residual, odd), torch.nn.functional.linear(residual, odd))
        ret[rank] = (ok, refused, float((residual - want).abs().max()))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_sharded_layer_equals_unsharded(world):
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=_rank_main, args=(r, world, port, ret)) for r in range(world)]
    for pr in procs:
        pr.start()
    for pr in procs:
        pr.join(timeout=240)
        assert pr.exitcode == 0, f"rank exited with {pr.exitcode}"
    for r in range(world):
        ok, refused, err = ret[r]
        assert ok, f"rank {r}: sharded result differs from the unsharded oracle (max |d| = {err})"
        assert refused


def test_oracle_tp_restatement_matches():
    cfg, full = _model_sd(hidden=128, heads=4, ffn=256)
    from torch_int.models.tensor_parallel import TensorParallel
    g = torch.Generator().manual_seed(12)
    hidden = torch.randn((1, 32, 128), generator=g)
    mask = O.causal_mask(1, 32, 32)
    want, _ = OM.decoder_layer(full, "model.decoder.layers.0", hidden, mask, 4)
    for world in (1, 2, 4):
        shards = [TensorParallel(world, r).shard_state_dict(full) for r in range(world)]
        got = OM.decoder_layer_tp(shards, "model.decoder.layers.0", hidden, mask, 4)
        assert torch.equal(got, want), f"tp={world}"


def test_single_rank_context_is_a_no_op():
    from torch_int.models.tensor_parallel import TensorParallel
    tp = TensorParallel.single()
    t = torch.arange(6, dtype=torch.int32)
    assert tp.all_reduce_int32(t) is t
    sd = {"x.q_proj.weight": torch.zeros(4, 4)}
    assert tp.shard_state_dict(sd)["x.q_proj.weight"].shape == (4, 4)


# --------------------------------------------------------------------------- the product model on CPU ranks
def _model_rank_main(rank, world, port, ret):
    """The PRODUCT's tensor-parallel model code (torch_int.models.opt with a TensorParallel context) on
    gloo ranks: the extension is replaced by the oracle-backed stand-ins of tests/cpu_ops_stub.py and CUDA
    streams by no-ops, so the Python of both layer loops runs - the all-reduce form (short inputs, decode
    steps) and the pipelined reduce-scatter / LayerNorm-on-my-rows / all-gather form with its collective
    fallback (the peer-memory exchange itself needs GPUs) - and must reproduce the single-rank oracle."""
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import cpu_ops_stub as stub
        from torch_int.models.opt import Int8OPTConfig
        from torch_int.models.random_init import random_int8_opt
        from torch_int.models.tensor_parallel import TensorParallel
        torch.set_num_threads(1)
        stub.install()
        stub.install_serial_streams()
        cfg = Int8OPTConfig(vocab_size=64, hidden_size=256, num_hidden_layers=2, ffn_dim=512,
                            num_attention_heads=4, max_position_embeddings=64)
        whole = random_int8_opt(cfg, seed=5, device="cpu")                 # the same model, unsplit
        full_sd = {k: v.detach() for k, v in whole.state_dict().items()}
        tp = TensorParallel.from_world()
        tp.use_peer_memory = False
        model = random_int8_opt(cfg, seed=5, device="cpu", tp=tp)
        ids = torch.randint(2, 64, (4, 24), generator=torch.Generator().manual_seed(8))
        want, _ = OM.causal_lm_logits(full_sd, cfg, ids)
        checks = {}
        # all-reduce form (fewer tokens than min_pipeline_tokens)
        assert tp.plan_chunks(4, 24) == 0
        checks["all_reduce"] = torch.equal(model(ids).logits, want)
        # pipelined form: 4 sequences -> max_chunks groups; rows per group divisible by the ranks
        tp.min_pipeline_tokens = 1
        tp.max_chunks = 2
        assert tp.plan_chunks(4, 24) == 2
        checks["pipelined_2_groups"] = torch.equal(model(ids).logits, want)
        tp.max_chunks = 4
        assert tp.plan_chunks(4, 24) == 4
        checks["pipelined_4_groups"] = torch.equal(model(ids).logits, want)
        # the same with the timeline spans switched on (events are no-ops here; only the plumbing runs)
        from torch_int.models.tensor_parallel import StreamTrace
        tp.trace = StreamTrace()
        checks["traced"] = torch.equal(model(ids).logits, want)
        names = {(name, row) for name, row, *_ in tp.trace.spans}
        checks["trace_rows"] = names == {("attention+out_proj", "compute"), ("fc1+fc2", "compute"),
                                         ("nccl", "exchange.copy")}
        checks["trace_count"] = len(tp.trace.spans) == 2 * 2 * 4 * 2      # layers x phases x groups x (compute, exchange)
        tp.trace = None
        # vocabulary-parallel head on top of the pipelined loop
        tp.vocab_parallel = True
        checks["vocab_parallel"] = torch.allclose(model(ids).logits, want, rtol=1e-5, atol=1e-5)
        tp.vocab_parallel = False
        # cache + decode steps under tensor parallelism (decode steps use the all-reduce form)
        dec = model.model.decoder
        cache = model.new_cache(4, 32)
        model(ids[:, :20], past_key_values=cache, use_cache=True)
        step = dec.decode_step(ids[:, 20:21], cache)[:, -1]
        checks["decode_step"] = torch.equal(step, OM.decoder(full_sd, cfg, ids[:, :21])[0][:, -1])
        ret[rank] = checks
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_product_model_on_cpu_ranks(world):
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=_model_rank_main, args=(r, world, port, ret)) for r in range(world)]
    for pr in procs:
        pr.start()
    for pr in procs:
        pr.join(timeout=300)
        assert pr.exitcode == 0, f"rank exited with {pr.exitcode}"
    for r in range(world):
        assert all(ret[r].values()), f"rank {r}: {ret[r]}"


# --------------------------------------------------------------- collective decisions of the exchange
def _decision_rank_main(rank, world, port, ret):
    """Host logic that decides between the peer-memory exchange and NCCL: a failure seen by ONE rank
    (allocation, or a barrier whose wait ran out) must move ALL ranks, at the same point."""
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import cpu_ops_stub as stub
        import torch_int.models.tensor_parallel as tpm
        from torch_int.models.tensor_parallel import PeerWorkspace, TensorParallel
        checks = {}
        # 1. the allocation fails on rank 1 only: every rank gets None and switches to NCCL together
        tp = TensorParallel.from_world()
        calls = []

        def allocate(self, tp_, chunks, mc, e, device):
            calls.append("allocate")
            if tp_.rank == 1:
                raise RuntimeError("out of symmetric memory (injected)")
            self.tp = tp_

        def preflight(self):
            calls.append("preflight")

        PeerWorkspace._allocate, PeerWorkspace._map_and_preflight = allocate, preflight
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")
            ws = tp.peer_workspace(2, 64, 32, "cpu")
        checks["all_fall_back"] = ws is None and tp.use_peer_memory is False
        checks["no_rank_went_on_alone"] = "preflight" not in calls     # nobody entered the next collective phase
        # 2. the preflight fails on the last rank only
        tp = TensorParallel.from_world()
        calls.clear()

        def allocate_ok(self, tp_, chunks, mc, e, device):
            self.tp = tp_

        def preflight_bad(self):
            if self.tp.rank == world - 1:
                raise RuntimeError("peer-memory barrier preflight failed (injected)")

        PeerWorkspace._allocate, PeerWorkspace._map_and_preflight = allocate_ok, preflight_bad
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")
            checks["preflight_failure_is_collective"] = tp.peer_workspace(2, 64, 32, "cpu") is None and not tp.use_peer_memory
        # 3. everything fine: all ranks get a workspace, cached under its key
        tp = TensorParallel.from_world()
        PeerWorkspace._map_and_preflight = lambda self: None
        ws = tp.peer_workspace(2, 64, 32, "cpu")
        checks["workspace"] = ws is not None and tp.peer_workspace(2, 64, 32, "cpu") is ws and ws.checked is False
        # 4. after a pass, rank 0 alone finds status 105: all ranks raise, drop the workspace, use NCCL next
        stub.device_status = lambda reset=False: 105 if rank == 0 else 0
        import torch_int
        torch_int._CUDA = stub                       # check_exchange imports the module lazily
        import sys
        sys.modules["torch_int._CUDA"] = stub
        raised = False
        try:
            tp.check_exchange(ws, "cpu")
        except RuntimeError as exc:
            raised = "status 105" in str(exc)
        checks["status_is_agreed"] = raised and tp.use_peer_memory is False and not tp._workspaces and ws.checked
        # 5. a clean status marks the workspace as checked and keeps the peer path
        tp = TensorParallel.from_world()
        ws = tp.peer_workspace(2, 64, 32, "cpu")
        stub.device_status = lambda reset=False: 0
        tp.check_exchange(ws, "cpu")
        checks["clean_pass"] = ws.checked and tp.use_peer_memory and tp.peer_workspace(2, 64, 32, "cpu") is ws
        ret[rank] = checks
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_peer_or_nccl_is_decided_by_all_ranks_together(world):
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=_decision_rank_main, args=(r, world, port, ret)) for r in range(world)]
    for pr in procs:
        pr.start()
    for pr in procs:
        pr.join(timeout=120)
        assert pr.exitcode == 0, f"rank exited with {pr.exitcode}"
    for r in range(world):
        assert all(ret[r].values()), f"rank {r}: {ret[r]}"
