"""CPU restatement of the three gather/copy operators, written as the slicing
loops of the reference's own kernel tests.  TEST INFRASTRUCTURE ONLY
(see ``oracle/__init__.py``).
"""
from __future__ import annotations

import torch


def gather_copy_vectors(key_src, key_dst, value_src, value_dst, src_meta, dst_meta, indices,
                        copy_start: int, copy_num: int) -> None:
    """library/retroinfer/test/test_gather_copy.py:233-237 — rows
    ``indices[g, copy_start:copy_start+copy_num]`` of keys, values and the per-row
    metadata are copied to the front of the destination buffers (in place)."""
    groups = key_src.shape[0]
    sel = indices[:, copy_start:copy_start + copy_num].long()
    for g in range(groups):
        key_dst.view(groups, -1, key_src.shape[-1])[g, :copy_num] = key_src[g, sel[g]]
        value_dst.view(groups, -1, key_src.shape[-1])[g, :copy_num] = value_src[g, sel[g]]
        dst_meta.view(groups, -1)[g, :copy_num] = src_meta[g, sel[g]]


def gather_copy_and_concat(key_src1, key_src2, key_src3, key_dst, value_src1, value_src2, value_src3,
                           value_dst, idx2, size2, dst2, chunks2, idx3, size3, dst3, chunks3,
                           valid_lengths, copy_vectors1: int) -> None:
    """library/retroinfer/test/test_gather_copy.py:110-127 — destination rows are
    ``src1[:copy_vectors1]`` ‖ for each listed unit of src2 (vector-level start index)
    its first ``size`` rows ‖ for each listed unit of src3 (unit-level index) its first
    ``size`` rows; ``valid_lengths[g]`` is the number of rows written.

    ``dst2``/``dst3`` are the exclusive running sums of the sizes, as the kernel
    consumes them (copy_kernel.cuh:255-262)."""
    groups = key_src1.shape[0]
    d = key_src1.shape[-1]
    kd = key_dst.view(groups, -1, d)
    vd = value_dst.view(groups, -1, d)
    for g in range(groups):
        kd[g, :copy_vectors1] = key_src1[g, :copy_vectors1]
        vd[g, :copy_vectors1] = value_src1[g, :copy_vectors1]
        n = copy_vectors1
        for j in range(int(chunks2[g])):
            s, m = int(idx2[g, j]), int(size2[g, j])
            kd[g, n:n + m] = key_src2[g, s:s + m]
            vd[g, n:n + m] = value_src2[g, s:s + m]
            n += m
        for j in range(int(chunks3[g])):
            u, m = int(idx3[g, j]), int(size3[g, j])
            kd[g, n:n + m] = key_src3[g, u, :m]
            vd[g, n:n + m] = value_src3[g, u, :m]
            n += m
        valid_lengths[g] = n


def gather_copy_and_scatter(key_src, key_dst, value_src, value_dst, src_idx, sizes, dst_idx, chunks,
                            copy_start: int) -> None:
    """library/retroinfer/test/test_gather_copy.py:190-194 — for each listed unit,
    ``size`` rows starting at ``copy_start + src_idx`` of the source go to the first
    rows of destination unit ``dst_idx`` (in place)."""
    groups = key_src.shape[0]
    d = key_src.shape[-1]
    ks = key_src.view(groups, -1, d)
    vs = value_src.view(groups, -1, d)
    for g in range(groups):
        for j in range(int(chunks[g])):
            s, m, u = copy_start + int(src_idx[g, j]), int(sizes[g, j]), int(dst_idx[g, j])
            key_dst[g, u, :m] = ks[g, s:s + m]
            value_dst[g, u, :m] = vs[g, s:s + m]
