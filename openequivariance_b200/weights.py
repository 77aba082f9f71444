"""Weight layout of the kernels ("oeq order") and its map to e3nn order.

e3nn flattens weights instruction-major, each instruction's block row-major in
its ``path_shape``: ``[u][v]`` for "uvu", ``[u][v][w]`` for "uvw".  The
kernels consume the layout the reference's kernels consume (reference:
openequivariance/implementations/ComputationSchedule.py:146-230 for the
32-wide splitting, :427-471 for the permutation): every multiplicity axis is
cut into chunks of at most 32; the chunks of one instruction are visited with
the u-chunk outermost, then the v-chunk, then (uvw only) the w-chunk; and each
chunk is stored with its first two axes swapped, ``[v][u]`` or ``[v][u][w]``.
For "uvu" with every second-input multiplicity equal to 1 the two orders are
identical.

``oeq_from_e3nn_index(problem)`` returns the gather index ``g`` with
``w_oeq[..., t] = w_e3nn[..., g[t]]``.
"""

from __future__ import annotations

from math import prod

import numpy as np

CHUNK = 32


def _chunks(extent: int):
    return [slice(lo, min(lo + CHUNK, extent)) for lo in range(0, extent, CHUNK)]


def oeq_from_e3nn_index(problem) -> np.ndarray:
    """Gather index (int64, length ``weight_numel``) from e3nn order to oeq order."""
    pieces = []
    start = 0
    for ins in problem.instructions:
        if not ins.has_weight:
            continue
        shape = ins.path_shape
        block = np.arange(start, start + prod(shape), dtype=np.int64).reshape(shape)
        start += prod(shape)
        mode = ins.connection_mode
        if mode == "uvu":
            for us in _chunks(shape[0]):
                for vs in _chunks(shape[1]):
                    pieces.append(block[us, vs].T.ravel())
        elif mode == "uvw":
            for us in _chunks(shape[0]):
                for vs in _chunks(shape[1]):
                    for ws in _chunks(shape[2]):
                        pieces.append(block[us, vs, ws].transpose(1, 0, 2).ravel())
        else:
            raise ValueError(f"weight layout is defined for 'uvu' and 'uvw' only, got {mode!r}")
    if not pieces:
        return np.zeros(0, dtype=np.int64)
    return np.concatenate(pieces)


def reorder_weights(problem, weights_in, weights_out, direction: str, has_batch_dim: bool):
    """Fill ``weights_out`` with ``weights_in`` permuted between the two layouts.

    ``direction="forward"`` maps e3nn order to oeq order, ``"backward"`` the
    inverse.  Works on numpy arrays and torch tensors (last axis = weights;
    a leading batch axis when ``has_batch_dim``), mirroring the call
    convention ``reorder(input, output, has_batch_dim)`` of the reference
    (reference: openequivariance/implementations/LoopUnrollTP.py:65-68).
    """
    assert direction in ("forward", "backward")
    gather = oeq_from_e3nn_index(problem)
    if direction == "backward":
        inverse = np.empty_like(gather)
        inverse[gather] = np.arange(gather.size, dtype=np.int64)
        gather = inverse
    if isinstance(weights_in, np.ndarray):
        index = gather
    else:
        import torch
        index = torch.as_tensor(gather, device=weights_in.device)
    if has_batch_dim:
        weights_out[:, :] = weights_in[:, index]
    else:
        weights_out[:] = weights_in[index]
    return weights_out
