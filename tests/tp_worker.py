"""Worker for the 2-GPU tensor-parallel test: one process per GPU under torchrun."""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main():
    import torch
    import torch.distributed as dist
    from lighterpp_b200 import engine as E, synth
    from oracle.oracle import Oracle
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dist.init_process_group("gloo")
    ids = [E.nccl_unique_id() if rank == 0 else None]
    dist.broadcast_object_list(ids, src=0)
    name = sys.argv[1]
    c, dt, tied, seed, T = synth.named(name)
    mode = sys.argv[2] if len(sys.argv) > 2 else "peer"
    eng = E.Engine(c, dt, "f16", device=local, tp_rank=rank, tp_size=world, nccl_id=ids[0],
                   flags=E.FLAG_TP_NCCL if mode == "nccl" else 0)
    if mode == "peer":
        # the exchange fused into the residual GEMVs: every rank maps every rank's receive buffer
        handles = [None] * world
        dist.all_gather_object(handles, eng.tp_export())
        eng.tp_connect(handles)
    eng.load_weights(T)  # full tensors in, this rank's share kept
    m = Oracle().model(c, synth.as_f32(T))
    toks = synth.prompt_tokens(c.vocab_size, 8, seed)
    worst = 0.0
    for pos, t in enumerate(toks):
        ref = m.step_logits(int(t), pos)
        got = eng.step_logits(int(t), pos)
        worst = max(worst, float(np.abs(ref - got).max()))
        assert worst < 2e-2
    out, _ = eng.decode(int(toks[0]), 0, 16, 0.9, 1.1, [1], 64, np.linspace(0.05, 0.95, 16, dtype=np.float32))
    gathered = [None] * world
    dist.all_gather_object(gathered, out.tolist())
    assert all(g == gathered[0] for g in gathered), gathered
    dist.barrier()
    if rank == 0:
        print(f"TP_OK world={world} mode={mode} worst={worst:.2e} tokens={out.tolist()}")
    eng.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
