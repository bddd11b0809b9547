"""Worker of tests/test_gpu_tp_decoder.py: one rank of a column-parallel decode harness.  Started by
torch.distributed.run; rank 0 writes the generated tokens to the file given as argument."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    out_path = sys.argv[1]
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    from cherryq_b200 import decoder as D
    cfg = D.DecoderConfig(n_layers=2, hidden=256, n_heads=4, n_kv_heads=2, ffn=512, vocab=1000, bits=4, group=128,
                          cherry_fraction=1 / 32, max_seq=128)
    model = D.CherryDecoder(cfg, device=dev, seed=5, tp_group=dist.group.WORLD)
    prompt = torch.randint(0, cfg.vocab, (40,), device=dev, generator=torch.Generator(device=dev).manual_seed(1))
    model.prefill(prompt)
    eager = model.generate(12, use_graph=False)
    model.prefill(prompt)
    graphed = model.generate(12, use_graph=True)
    torch.cuda.synchronize()
    if dist.get_rank() == 0:
        torch.save({"eager": eager.cpu(), "graphed": graphed.cpu()}, out_path)
    dist.barrier()
    torch.cuda.synchronize()
    sys.stdout.flush()
    os._exit(0)          # (no communicator teardown under live graphs that hold NCCL kernels)


if __name__ == "__main__":
    main()
