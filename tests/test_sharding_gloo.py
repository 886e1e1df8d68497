"""The N > 1 path on CPU: two gloo ranks, no GPU.  Each rank seeds the generator alike, plans
the whole batch (parameter draw + broadcast + slice bounds) and keeps its own slice; gathered
back, the slices must tile the single-process plan exactly, with whole videos per rank."""
import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

MEAN, STD = (0.485, 0.456, 0.406), (0.229, 0.224, 0.225)


def _make():
    import triton_augment_b200 as ta
    return ta, ta.TritonFusedAugment(crop_size=12, horizontal_flip_p=0.5, degrees=15, translate=(0.1, 0.1),
                                     scale=(0.9, 1.1), shear=5, brightness=0.2, contrast=0.2, saturation=0.2,
                                     grayscale_p=0.3, mean=MEAN, std=STD, same_on_frame=True)


def _tensor_params(spread):
    return [p.float().reshape(p.shape[0], -1) for p in spread if isinstance(p, torch.Tensor)]


def _worker(rank, world, port, shape, result_path):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        ta, aug = _make()
        sharder = ta.ShardedAugment.for_rank(aug, rank, world, device=torch.device("cuda", 0))   # device is not touched
        torch.manual_seed(1234)
        lay, spread, bounds = sharder.plan(shape, torch.device("cpu"))
        start, stop = bounds[rank]
        mine = torch.cat(_tensor_params(ta.multi_gpu.slice_params(spread, start, stop)), dim=1)
        sizes = [torch.zeros(1, dtype=torch.long) for _ in range(world)]
        dist.all_gather(sizes, torch.tensor([mine.shape[0]]))
        gathered = [torch.zeros(int(s), mine.shape[1]) for s in sizes]
        for r in range(world):                       # ragged gather: broadcast each rank's slice
            buf = mine if r == rank else gathered[r]
            dist.broadcast(buf, src=r)
            gathered[r] = buf
        if rank == 0:
            torch.manual_seed(1234)
            _, full, _ = ta.ShardedAugment(aug, [torch.device("cuda", 0)]).plan(shape, torch.device("cpu"))
            whole = torch.cat(_tensor_params(full), dim=1)
            ok = torch.equal(torch.cat(gathered), whole)
            frames = shape[1] if len(shape) == 5 else 1
            ok = ok and all((b - a) % frames == 0 for a, b in bounds) and bounds[-1][1] == whole.shape[0]
            with open(result_path, "w") as f:
                f.write("ok" if ok else "mismatch")
        dist.barrier()
    finally:
        dist.destroy_process_group()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _run(shape, tmp_path):
    result = str(tmp_path / "result.txt")
    mp.spawn(_worker, args=(2, _free_port(), shape, result), nprocs=2, join=True)
    assert open(result).read() == "ok"


def test_two_ranks_tile_the_image_batch(tmp_path):
    _run((11, 3, 20, 24), tmp_path)


def test_two_ranks_keep_videos_whole(tmp_path):
    _run((5, 4, 3, 20, 24), tmp_path)
