"""Generates tests/golden/reference_vectors.npz from the REFERENCE's own CUDA kernels.

Run on a machine with a GPU after `python oracle/build_ref.py` built oracle/_ref/ from the
reference tree:

    python tests/golden/make_golden.py [out.npz]
    python tests/golden/make_golden.py --kdtree [out.npz]     # reference_vectors_kdtree.npz

Every vector is an output of the unmodified reference implementation (radius_graph_pbc_cuda_impl_ex,
sfc_partition_cuda_impl, extract_halo_info_cuda_impl, filter_edges_to_radius_cuda_impl) on seeded
inputs that the CPU tests regenerate with the same code (`cases()` below).  Edge sets are stored in
canonical order (dst, src, shift) so that the file does not depend on the kernels' emission order.
"""

import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)


def cases():
    """name -> (pos, cell, pbc, radius, targets or None); all float32."""
    out = {}
    rng = np.random.default_rng(4242)

    def cubic(n, box):
        return (rng.random((n, 3)) * box).astype(np.float32), (np.eye(3) * box).astype(np.float32)

    p, c = cubic(100, 20.0)
    out["cubic100"] = (p, c, [True, True, True], 5.0, None)
    p, c = cubic(30, 8.0)
    out["multi_image"] = (p, c, [True, True, True], 6.0, None)
    p, c = cubic(5, 2.5)
    out["tiny_box"] = (p, c, [True, True, True], 6.0, None)
    cell = np.array([[12.0, 0.0, 0.0], [2.5, 11.0, 0.0], [1.5, -2.0, 13.0]], np.float32)
    out["triclinic"] = ((rng.random((200, 3)) @ cell.astype(np.float64)).astype(np.float32), cell, [True, True, True], 5.0, None)
    p, c = cubic(150, 14.0)
    out["pbc_xy"] = (p, c, [True, True, False], 4.5, None)
    out["no_pbc"] = (p, c, [False, False, False], 4.5, None)
    out["unwrapped"] = (((rng.random((200, 3)) - 0.5) * 60.0).astype(np.float32), (np.eye(3) * 15.0).astype(np.float32),
                        [True, True, True], 4.0, None)
    p, c = cubic(400, 25.0)
    out["subset"] = (p, c, [True, True, True], 5.0, rng.permutation(400)[:150].astype(np.int64))
    out["single_atom"] = (np.array([[2.5, 2.5, 2.5]], np.float32), (np.eye(3) * 5.0).astype(np.float32), [True, True, True], 6.0, None)
    return out


def sfc_case():
    rng = np.random.default_rng(777)
    pos = (rng.random((3000, 3)) * 50.0 - 5.0).astype(np.float32)
    w = rng.integers(1, 400, 3000).astype(np.int64)
    return pos, w


def halo_case():
    rng = np.random.default_rng(13)
    pos = (rng.random((4000, 3)) * 40.0).astype(np.float32)
    cell = (np.eye(3) * 40.0).astype(np.float32)
    W = 4
    pid = np.minimum((pos[:, 0] / (40.0 / W)).astype(np.int64), W - 1)
    return pos, cell, pid, W


def kdtree_case():
    """3000 positions whose coordinates are distinct per axis (the reference's sort leaves ties open) and
    weights whose sums stay far below 2**24 (its float32 cumulative sum is exact there)."""
    rng = np.random.default_rng(2024)
    n = 3000
    pos = np.empty((n, 3), dtype=np.float32)
    for d, scale in enumerate((30.0, 12.0, 20.0)):
        ramp = (np.arange(n, dtype=np.float64) + rng.random(n) * 0.5) * (scale / n)
        pos[:, d] = rng.permutation(ramp).astype(np.float32)
        assert np.unique(pos[:, d]).size == n
    w = rng.integers(1, 60, n).astype(np.int64)
    return pos, w


def main_kdtree(path):
    """tests/golden/reference_vectors_kdtree.npz: labels of the reference's kdtree_bisect_cuda_impl."""
    import torch

    from oracle import build_ref

    assert build_ref.load(), "oracle/_ref/libdynamis_ref.so is missing: run python oracle/build_ref.py"
    ref = torch.ops.dynamis_ref
    dev = torch.device("cuda:0")
    pos, w = kdtree_case()
    tp, tw = torch.as_tensor(pos, device=dev), torch.as_tensor(w, device=dev)
    out = {}
    for W in (2, 3, 5, 8, 13):
        out[f"kd_W{W}"] = ref.kdtree_partition(tp, None, W).cpu().numpy().astype(np.int16)
        out[f"kd_weighted_W{W}"] = ref.kdtree_partition(tp, tw, W).cpu().numpy().astype(np.int16)
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes,", len(out), "arrays")


def main():
    import torch

    from oracle import build_ref
    from oracle import cpu_oracle as O

    assert build_ref.load(), "oracle/_ref/libdynamis_ref.so is missing: run python oracle/build_ref.py"
    ref = torch.ops.dynamis_ref
    dev = torch.device("cuda:0")
    out = {}
    for name, (pos, cell, pbc, r, targets) in cases().items():
        tt = torch.as_tensor(targets, device=dev) if targets is not None else None
        ei, cs, nn, counts = ref.radius_graph(torch.as_tensor(pos, device=dev), torch.as_tensor(cell, device=dev),
                                              torch.tensor(pbc, device=dev), float(r), tt, False)
        ei = ei.cpu().numpy()
        out[f"rg_{name}_edges"] = O.canonical_edges(ei[0], ei[1], cs.cpu().numpy()).astype(np.int32)
        out[f"rg_{name}_counts"] = counts.cpu().numpy()
    pos, w = sfc_case()
    tp, tw = torch.as_tensor(pos, device=dev), torch.as_tensor(w, device=dev)
    for W in (2, 8, 13):
        out[f"sfc_morton_W{W}"] = ref.sfc_partition(tp, None, W, 0).cpu().numpy().astype(np.int16)
        out[f"sfc_morton_weighted_W{W}"] = ref.sfc_partition(tp, tw, W, 0).cpu().numpy().astype(np.int16)
        out[f"sfc_hilbert_counts_W{W}"] = torch.bincount(ref.sfc_partition(tp, None, W, 1), minlength=W).cpu().numpy()
    pos, cell, pid, W = halo_case()
    tp, tc, tpid = torch.as_tensor(pos, device=dev), torch.as_tensor(cell, device=dev), torch.as_tensor(pid, device=dev)
    for rank in range(W):
        mine = torch.nonzero(tpid == rank).squeeze(-1)
        ei, cs, _, _ = ref.radius_graph(tp, tc, torch.tensor([True] * 3, device=dev), float(np.float32(6.5)), mine, False)
        so, sl, ro, rg, im, ra = ref.extract_halo_info(ei, tpid, mine, rank, W, pos.shape[0])
        out[f"halo_r{rank}_send_offsets"] = so.cpu().numpy()
        out[f"halo_r{rank}_send_local"] = sl.cpu().numpy().astype(np.int32)
        out[f"halo_r{rank}_recv_offsets"] = ro.cpu().numpy()
        out[f"halo_r{rank}_recv_atom"] = ra.cpu().numpy().astype(np.int32)
        out[f"halo_r{rank}_interior"] = np.packbits(im.cpu().numpy())
        fe, fs = ref.filter_edges(ei, cs, tp, tc, 6.0)
        out[f"halo_r{rank}_filtered_digest"] = np.array(O.edge_set_digest(fe[0].cpu().numpy(), fe[1].cpu().numpy(), fs.cpu().numpy()),
                                                        dtype=np.uint64)
    path = sys.argv[1] if len(sys.argv) > 1 else os.path.join(ROOT, "tests", "golden", "reference_vectors.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes,", len(out), "arrays")


if __name__ == "__main__":
    if "--kdtree" in sys.argv:
        rest = [a for a in sys.argv[1:] if a != "--kdtree"]
        main_kdtree(rest[0] if rest else os.path.join(ROOT, "tests", "golden", "reference_vectors_kdtree.npz"))
    else:
        main()
