"""One rank of a tensor-parallel run (launched by tests/test_gpu_tp.py with torch.distributed.run).

mode "parity":  small Llama-shape model sharded over WORLD_SIZE GPUs; prompt + greedy steps, every rank checks its
                tokens against the CPU oracle of the unsharded model.
mode "parity_lfm2": the same for a small LFM2-like model: short-conv layers with their channels split across ranks
                (three-section column shard of the B|C|x projection) next to attention layers with QK-norm.
mode "prompt" / "prompt_lfm2": a 150-token prompt goes through the chunked path (tensor-core products on each rank's
                shard, partial rows summed across ranks per chunk), then greedy steps; tokens against the oracle.
mode "timeout": the last rank stays alive but never decodes; the others' bounded waits must expire and
                surface as SWLM_ERR_TIMEOUT. No rank exits, traps or faults while kernels are in flight.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
from conftest import load_package  # noqa: E402
import oracle_binding  # noqa: E402


def main():
    import torch
    import torch.distributed as dist

    mode = sys.argv[1]
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo")  # host-side plumbing only; the data path is the library's own kernels
    pkg = load_package()
    batch = 2 if mode == "parity2" else 1
    max_seq = 256 if mode.startswith("prompt") else 96
    if mode in ("parity_lfm2", "prompt_lfm2"):
        cfg = pkg.ModelConfig("lfm2", hidden=512, intermediate=1024, layers=5, heads=8, kv_heads=4, head_dim=64,
                              vocab=4096, norm_eps=1e-5, rope_theta=1000000.0, conv_kernel=3, attention_layers=[1, 3],
                              max_seq=max_seq, max_batch=batch)
    elif world > 4:   # one KV head per rank at 8 ranks
        cfg = pkg.ModelConfig("llama", hidden=1024, intermediate=2048, layers=3, heads=16, kv_heads=8, head_dim=64,
                              vocab=4096, max_seq=max_seq, max_batch=batch)
    else:
        cfg = pkg.ModelConfig("llama", hidden=512, intermediate=1536, layers=3, heads=8, kv_heads=4, head_dim=64,
                              vocab=4096, max_seq=max_seq, max_batch=batch)
    builder = pkg.DispatchPlanBuilder(cfg)
    weights = pkg.synth_model_weights(builder, seed=5)
    store = pkg.WeightStore(rank, tp_rank=rank, tp_size=world)
    model = pkg.load_model(store, builder, weights)
    pkg.tp.attach(model, dist)
    long_prompt = mode.startswith("prompt")
    prompt = np.random.default_rng(2).integers(0, cfg.vocab, size=(batch, 150 if long_prompt else 6), dtype=np.int32)

    if mode.startswith("parity") or long_prompt:
        om = oracle_binding.Oracle(os.path.join(os.path.dirname(HERE), "oracle", "liboracle.so")).model(cfg.buffers_desc())
        om.load(builder, weights)
        if long_prompt:
            model.set_prefill_chunk(64)
        before = model.launches
        g, o = model.prefill(prompt), om.prefill(prompt)
        if long_prompt:   # far fewer launches than 150 decode steps: the prompt went through the chunked path
            assert model.launches - before < 40 * model.launches_per_step, (model.launches - before, model.launches_per_step)
        bad = 0
        for _ in range(24):
            bad += int((g != o).sum())
            g, o = model.decode(o), om.decode(o)
        assert pkg.tp.status(model) == 0
        assert "push" in model.describe() and "allreduce+" in model.describe()
        # every rank must have produced the same tokens as the oracle (ties aside)
        assert bad <= 1, f"rank {rank}: {bad} token mismatches"
        more = model.decode_n(o, 8)
        gathered = [None] * world
        dist.all_gather_object(gathered, more.tolist())
        assert all(x == gathered[0] for x in gathered), "ranks diverged"
        print(f"TP_OK rank={rank} mismatches={bad}", flush=True)
    elif mode == "timeout":
        if rank != world - 1:
            # the call that produces tokens reports the expired wait itself (status -5, tokens -1) ...
            status = 0
            try:
                model.prefill(prompt)
            except pkg.SwlmError as e:
                status = e.status
            assert status == -5, f"prefill: expected SWLM_ERR_TIMEOUT, got {status}"
            # ... and so does the explicit query
            st = pkg.tp.status(model)
            assert st == -5, f"expected SWLM_ERR_TIMEOUT, got {st}"
            print(f"TP_TIMEOUT_OK rank={rank}", flush=True)
        dist.barrier()  # the idle rank leaves only after the others have finished and synchronised
    dist.barrier()
    model.close()
    store.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
