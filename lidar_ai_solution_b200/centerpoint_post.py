"""CenterPoint head decode + rotated NMS on the device (ctypes over ``spconvb_cp_*``).

Host-side mirror of ``PostProcessCuda`` and of the per-task loop in ``CenterPoint::doinfer``
(CUDA-CenterPoint/include/postprocess.h:55-88, src/centerpoint.cpp:163-216): the six task
heads go in, a list of ``Bndbox`` rows ``[x, y, z, w, l, h, vx, vy, rt, id, score]`` comes
out, with no host synchronisation in between.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import cabi

# Params::task_num_stride and the class count of each nuScenes task head
# (CUDA-CenterPoint/include/common.h:58-60)
TASK_LABEL_OFFSET = (0, 1, 3, 5, 6, 8)
TASK_NUM_CLASSES = (1, 2, 2, 1, 2, 2)
HEAD_CHANNELS = {"reg": 2, "height": 1, "dim": 3, "rot": 2, "vel": 2}


def default_params(H=180, W=180, **overrides) -> cabi.CpParams:
    p = cabi.CpParams()
    cabi.lib().spconvb_cp_default_params(C.byref(p))
    p.H, p.W = H, W
    for k, v in overrides.items():
        cur = getattr(p, k)
        if hasattr(cur, "__len__"):
            for i, x in enumerate(v):
                cur[i] = x
        else:
            setattr(p, k, v)
    return p


class PostProcess:
    """Reusable post-processor: owns the workspace and the output list."""

    def __init__(self, params: cabi.CpParams | None = None, num_tasks=6, device="cuda"):
        self.lib = cabi.lib()
        self.params = params or default_params()
        self.num_tasks = num_tasks
        nbytes = self.lib.spconvb_cp_workspace_bytes(C.byref(self.params), num_tasks)
        if nbytes == 0:
            raise ValueError("bad post-processing parameters")
        self.workspace = torch.zeros(nbytes, dtype=torch.uint8, device=device)
        self.boxes = torch.zeros((num_tasks * self.params.nms_post_max, 11), dtype=torch.float32,
                                 device=device)
        self.count = torch.zeros(1, dtype=torch.int32, device=device)
        self._heads = (cabi.CpHead * num_tasks)()
        self._keep = None

    def run(self, heads, label_offsets=TASK_LABEL_OFFSET, stream=None):
        """heads: one dict per task of contiguous cuda fp16 tensors ``reg height dim rot vel hm``
        shaped [C, H, W].  Enqueues the work; ``self.boxes[:self.count]`` holds the result once
        the stream has run."""
        assert len(heads) == self.num_tasks
        p = self.params
        for t, h in enumerate(heads):
            for k, ch in HEAD_CHANNELS.items():
                x = h[k]
                assert x.is_cuda and x.dtype == torch.float16 and x.is_contiguous()
                assert tuple(x.shape[-3:]) == (ch, p.H, p.W), (k, tuple(x.shape))
                setattr(self._heads[t], k, x.data_ptr())
            hm = h["hm"]
            assert hm.is_cuda and hm.dtype == torch.float16 and hm.is_contiguous()
            assert tuple(hm.shape[-2:]) == (p.H, p.W)
            self._heads[t].hm = hm.data_ptr()
            self._heads[t].num_classes = hm.shape[-3]
            self._heads[t].label_offset = label_offsets[t]
        self._keep = heads
        s = stream if stream is not None else torch.cuda.current_stream()
        cabi.check(self.lib.spconvb_cp_postprocess(
            self._heads, self.num_tasks, C.byref(p), self.workspace.data_ptr(),
            self.workspace.numel(), self.boxes.data_ptr(), self.count.data_ptr(),
            C.c_void_p(s.cuda_stream)), "cp_postprocess")

    def result(self):
        """Synchronises and returns the kept boxes [n, 11] (a copy)."""
        n = int(self.count.item())
        return self.boxes[:n].clone()

    def task_detections(self, task):
        """Ranked detections of one task before NMS, [n, 11] = x y z dx dy dz vx vy rot label
        score (synchronises)."""
        det, n = C.c_void_p(), C.c_void_p()
        cabi.check(self.lib.spconvb_cp_task_detections(
            C.byref(self.params), self.num_tasks, self.workspace.data_ptr(), task, C.byref(det),
            C.byref(n)), "cp_task_detections")
        base = self.workspace.data_ptr()
        cnt = int(self.workspace[n.value - base:n.value - base + 4].view(torch.int32).item())
        off = det.value - base
        return self.workspace[off:off + cnt * 44].view(torch.float32).reshape(cnt, 11).clone()


def rotated_iou(boxes_a, boxes_b):
    """Bird's-eye IoU of pairs of boxes [n, 7] = x y z dx dy dz angle (cuda float32)."""
    a = boxes_a.contiguous().float()
    b = boxes_b.contiguous().float()
    out = torch.empty(a.shape[0], dtype=torch.float32, device=a.device)
    cabi.check(cabi.lib().spconvb_cp_rotated_iou(
        a.data_ptr(), b.data_ptr(), a.shape[0], out.data_ptr(),
        C.c_void_p(torch.cuda.current_stream().cuda_stream)), "cp_rotated_iou")
    return out


def _main(argv=None):
    """Times one frame's post-processing (six task heads) as a CUDA-graph replay."""
    import argparse
    import json

    from . import scenes
    ap = argparse.ArgumentParser(description=_main.__doc__)
    ap.add_argument("--mean-logit", type=float, default=-6.0,
                    help="heat-map background level: -6 gives a few hundred candidates per task, "
                         "-3 several thousand")
    ap.add_argument("--iters", type=int, default=200)
    ap.add_argument("--seed", type=int, default=0)
    args = ap.parse_args(argv)
    heads = scenes.make_centerpoint_heads(args.seed, mean_logit=args.mean_logit)
    dev = [{k: torch.from_numpy(v).cuda() for k, v in h.items()} for h in heads]
    pp = PostProcess()
    pp.run(dev)
    torch.cuda.synchronize()
    stream = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(stream):
        with torch.cuda.graph(graph, stream=stream):
            pp.run(dev, stream=stream)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
    total = 0.0
    for i in range(args.iters + 5):
        flush.zero_()                       # heads come from HBM, not from a warm L2
        ev[0].record()
        graph.replay()
        ev[1].record()
        torch.cuda.synchronize()
        if i >= 5:
            total += ev[0].elapsed_time(ev[1])
    per_task = [int(pp.task_detections(t).shape[0]) for t in range(pp.num_tasks)]
    print(json.dumps({"what": "centerpoint decode + nms, 6 task heads, cuda graph replay",
                      "us_per_frame": round(1000.0 * total / args.iters, 2),
                      "candidates_per_task": per_task, "boxes_kept": int(pp.count.item()),
                      "launches_per_frame": 5, "host_syncs_per_frame": 0}))


if __name__ == "__main__":
    _main()
