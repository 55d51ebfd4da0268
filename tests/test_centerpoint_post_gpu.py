"""CenterPoint head decode + rotated NMS through the C ABI against the CPU restatement.

Integer results (which cells, their order, labels, which boxes survive NMS) must be identical.
Floating-point fields go through expf / atan2f / sinf / cosf, whose CUDA and libm versions may
differ by a few ulp, so they are compared with a relative tolerance of 1e-5; products and sums
round identically on both sides (no multiply-add contraction on either)."""
import numpy as np
import pytest

torch = pytest.importorskip("torch")

from lidar_ai_solution_b200 import scenes  # noqa: E402
from oracle import oracle as orc  # noqa: E402

pytestmark = pytest.mark.gpu

RTOL = 1e-5


def _post():
    from lidar_ai_solution_b200 import centerpoint_post
    return centerpoint_post


def _dev_heads(heads):
    return [{k: torch.from_numpy(v).cuda() for k, v in h.items()} for h in heads]


def _oracle_frame(heads, offsets, params=None):
    """Per task (detections, kept boxes, decision margin) of the restatement."""
    out = []
    for h, off in zip(heads, offsets):
        det, cells = orc.centerpoint_decode(h, params)
        boxes, kept, margin = orc.centerpoint_nms(det, off, params)
        out.append((det, boxes, margin))
    return out


def test_rotated_iou_matches_the_restatement():
    post = _post()
    rng = np.random.default_rng(0)
    n = 20000
    a = np.zeros((n, 7), np.float32)
    a[:, 0:2] = rng.uniform(-3, 3, (n, 2))
    a[:, 3:5] = np.exp(rng.normal(0.6, 0.4, (n, 2)))
    a[:, 5] = 1.5
    a[:, 6] = rng.uniform(-4, 4, n)
    b = a.copy()
    b[:, 0:2] += rng.normal(0, 1.2, (n, 2))
    b[:, 3:5] *= np.exp(rng.normal(0, 0.2, (n, 2))).astype(np.float32)
    b[:, 6] += rng.normal(0, 0.7, n).astype(np.float32)
    b[:50] = a[:50]                      # identical boxes
    b[50:100, 0] = a[50:100, 0] + 50.0   # far apart
    b[100:150, 6] = a[100:150, 6]        # same heading, shifted
    want = orc.rotated_iou(a, b)
    got = post.rotated_iou(torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda()).cpu().numpy()
    assert np.all(got[50:100] == 0.0) and np.allclose(got[:50], 1.0, atol=1e-4)
    assert 0.25 < float((want > 0.2).mean()) < 0.95   # the sample straddles the NMS threshold
    assert float(np.abs(got - want).max()) <= 2e-5


@pytest.mark.parametrize("mean_logit,seed", [(-6.0, 17), (-3.0, 22)])
def test_decode_and_nms_match_the_restatement(mean_logit, seed):
    """-6: a few hundred candidates per task (the sort alone); -3: several thousand, more than
    nms_pre_max_size, so the radix select chooses the best 1000 first."""
    post = _post()
    heads = scenes.make_centerpoint_heads(seed, mean_logit=mean_logit)
    ref = _oracle_frame(heads, post.TASK_LABEL_OFFSET)
    pp = post.PostProcess()
    pp.run(_dev_heads(heads))
    got = pp.result().cpu().numpy()
    sizes = []
    for t, (det, boxes, margin) in enumerate(ref):
        d = pp.task_detections(t).cpu().numpy()
        sizes.append(len(det))
        assert d.shape == det.shape, "task %d: %d detections, oracle %d" % (t, len(d), len(det))
        assert np.array_equal(d[:, 9], det[:, 9])                       # labels
        assert np.array_equal(d[:, :3], det[:, :3])                     # centres: exact arithmetic
        assert np.array_equal(d[:, 6:8], det[:, 6:8])                   # velocities: copies
        assert np.allclose(d, det, rtol=RTOL, atol=1e-6)
        assert np.all(np.diff(d[:, 10]) <= 0)
        assert margin > 1e-4, "seed puts an IoU within rounding of the threshold; pick another"
    if mean_logit > -4:
        assert max(sizes) == 1000
    else:
        assert 50 < min(sizes) and max(sizes) < 1000
    want = np.concatenate([boxes for _, boxes, _ in ref])
    assert got.shape == want.shape
    assert np.array_equal(got[:, 9], want[:, 9])                        # class ids with offsets
    assert np.array_equal(got[:, :3], want[:, :3])                      # the same cells survive
    assert np.allclose(got, want, rtol=RTOL, atol=1e-6)
    per_task = [len(b) for _, b, _ in ref]
    assert max(per_task) <= 83 and sum(per_task) == len(got)


def test_empty_and_single_task_frames():
    post = _post()
    heads = scenes.make_centerpoint_heads(3, mean_logit=-12.0, objects=0)
    pp = post.PostProcess()
    pp.run(_dev_heads(heads))
    assert pp.result().shape == (0, 11)
    for t in range(6):
        assert pp.task_detections(t).shape == (0, 11)
    # one task, a small head, parameters away from the defaults
    heads = scenes.make_centerpoint_heads(4, H=64, W=96, mean_logit=-4.0, num_classes=(3,),
                                          objects=25)
    prm = dict(score_threshold=0.3, nms_iou_threshold=0.35, max_det=100, nms_post_max=20,
               pc_range=(-10.0, -20.0), post_center_range=(-30, -30, -3, 30, 30, 1))
    det, _ = orc.centerpoint_decode(heads[0], prm)
    boxes, kept, margin = orc.centerpoint_nms(det, 7, prm)
    assert margin > 1e-4 and len(det) == 100 and len(boxes) == 20
    cp = post.default_params(64, 96, **prm)
    pp = post.PostProcess(cp, num_tasks=1)
    pp.run(_dev_heads(heads), label_offsets=(7,))
    got = pp.result().cpu().numpy()
    assert np.array_equal(got[:, 9], boxes[:, 9]) and np.array_equal(got[:, :3], boxes[:, :3])
    assert np.allclose(got, boxes, rtol=RTOL, atol=1e-6)


@pytest.mark.parametrize("max_det", [64, 1000])
def test_tied_scores_rank_by_cell_index(max_det):
    """Heat maps with only five distinct logits: thousands of cells tie exactly, all pass the
    score filter, and the radix select has to cut inside a run of equal scores.  The ranking is
    then decided by the cell index, on the device as in the restatement."""
    post = _post()
    rng = np.random.default_rng(2)
    H, W = 64, 80
    heads = scenes.make_centerpoint_heads(2, H=H, W=W, num_classes=(2,), objects=0)
    heads[0]["hm"] = rng.choice(np.array([-1.0, -0.5, 0.0, 0.5, 2.0], np.float16), (2, H, W))
    prm = dict(max_det=max_det, nms_post_max=min(50, max_det), pc_range=(-20.0, -20.0),
               post_center_range=(-100, -100, -10, 100, 100, 10))
    det, cells = orc.centerpoint_decode(heads[0], prm)
    boxes, kept, margin = orc.centerpoint_nms(det, 2, prm)
    assert len(det) == max_det and margin > 1e-4
    assert len(np.unique(det[:, 10])) <= 3 and np.all(np.diff(cells[det[:, 10] == det[0, 10]]) > 0)
    pp = post.PostProcess(post.default_params(H, W, **prm), num_tasks=1)
    pp.run(_dev_heads(heads), label_offsets=(2,))
    d = pp.task_detections(0).cpu().numpy()
    assert np.array_equal(d[:, :3], det[:, :3]) and np.array_equal(d[:, 9:], det[:, 9:])
    got = pp.result().cpu().numpy()
    assert np.array_equal(got[:, 9], boxes[:, 9]) and np.array_equal(got[:, :3], boxes[:, :3])
    assert np.allclose(got, boxes, rtol=RTOL, atol=1e-6)


def test_postprocess_is_capturable_and_repeatable():
    """No host synchronisation inside: the call records into a CUDA graph; replays on new head
    values give the restatement's answer each time."""
    post = _post()
    pp = post.PostProcess()
    frames = [scenes.make_centerpoint_heads(s, mean_logit=-5.0) for s in (14, 22)]
    dev = _dev_heads(frames[0])
    pp.run(dev)                                 # warm-up outside capture
    torch.cuda.synchronize()
    stream = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(stream):
        with torch.cuda.graph(graph, stream=stream):
            pp.run(dev, stream=stream)
    for heads in (frames[1], frames[0], frames[1]):
        for d, h in zip(dev, heads):
            for k in d:
                d[k].copy_(torch.from_numpy(h[k]))
        torch.cuda.synchronize()
        graph.replay()
        torch.cuda.synchronize()
        got = pp.result().cpu().numpy()
        want = np.concatenate([b for _, b, _ in _oracle_frame(heads, post.TASK_LABEL_OFFSET)])
        assert got.shape == want.shape and np.array_equal(got[:, 9], want[:, 9])
        assert np.allclose(got, want, rtol=RTOL, atol=1e-6)


def test_bad_arguments_are_refused():
    post = _post()
    from lidar_ai_solution_b200 import cabi
    import ctypes as C
    lib = cabi.lib()
    p = post.default_params()
    heads = (cabi.CpHead * 1)()
    buf = torch.zeros(1 << 20, dtype=torch.uint8, device="cuda")
    out = torch.zeros(83 * 11, device="cuda")
    cnt = torch.zeros(1, dtype=torch.int32, device="cuda")
    # null head pointers
    assert lib.spconvb_cp_postprocess(heads, 1, C.byref(p), buf.data_ptr(), buf.numel(),
                                      out.data_ptr(), cnt.data_ptr(), None) == -1
    hs = _dev_heads(scenes.make_centerpoint_heads(0, num_classes=(1,)))
    for k in ("reg", "height", "dim", "rot", "vel", "hm"):
        setattr(heads[0], k, hs[0][k].data_ptr())
    heads[0].num_classes = 1
    # workspace too small
    assert lib.spconvb_cp_postprocess(heads, 1, C.byref(p), buf.data_ptr(), 4096,
                                      out.data_ptr(), cnt.data_ptr(), None) != 0
    p.max_det = 4096
    assert lib.spconvb_cp_postprocess(heads, 1, C.byref(p), buf.data_ptr(), buf.numel(),
                                      out.data_ptr(), cnt.data_ptr(), None) == -1
