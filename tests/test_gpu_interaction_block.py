"""A MACE-style interaction block trained for one step on energies and forces, on the GPU against the CPU oracle.

The reference validates its convolution inside MACE (test/mace_driver.py:124-140: a model whose interaction
blocks call the fused convolution, trained on energies and forces).  That model is not available here, so
this test builds the part of it that matters for the convolution: node features from species, edge attributes
from spherical harmonics of the edge vectors, per-edge weights from a radial network, the fused
gather - tensor product - scatter, an energy read out from the result, forces as the negative gradient of the
energy with respect to the positions (first derivatives of the convolution, kept in the graph), and one backward
pass of a loss on energy and forces (second derivatives of the convolution).  The same module runs with the
oracle's convolution on the CPU in float64; parameter gradients, forces and energy must agree.
"""
import math

import numpy as np
import pytest
import torch

import openequivariance_b200 as oeq
from openequivariance_b200.graph import spherical_harmonics
from oracle import tp_oracle as orc
from conftest import problem_by_name

pytestmark = pytest.mark.gpu


def neighbour_graph(positions, cutoff):
    """Both directions of every pair closer than ``cutoff`` (no self loops), in the reference's canonical
    (receiver, sender) order, with the sender-order permutation."""
    d = np.linalg.norm(positions[:, None, :] - positions[None, :, :], axis=-1)
    rows, cols = np.nonzero((d < cutoff) & (d > 0))
    rows, cols, order, perm = orc.coord_graph(rows.astype(np.int64), cols.astype(np.int64))
    return rows, cols, perm


class InteractionBlock(torch.nn.Module):
    def __init__(self, problem, lmax, n_species=3, n_radial=6, hidden=16, cutoff=1.0, seed=0):
        super().__init__()
        gen = torch.Generator().manual_seed(seed)
        rnd = lambda *shape: torch.randn(*shape, generator=gen, dtype=torch.float64)
        self.problem, self.lmax, self.cutoff = problem, lmax, cutoff
        self.embed = torch.nn.Parameter(rnd(n_species, problem.irreps_in1.dim))
        self.w1 = torch.nn.Parameter(rnd(n_radial, hidden) / math.sqrt(n_radial))
        self.w2 = torch.nn.Parameter(rnd(hidden, problem.weight_numel) / math.sqrt(hidden))
        self.readout = torch.nn.Parameter(rnd(problem.irreps_out.dim) / math.sqrt(problem.irreps_out.dim))
        self.register_buffer("freq", torch.arange(1, n_radial + 1, dtype=torch.float64) * math.pi / cutoff)

    def energy(self, positions, species, rows, cols, conv):
        vec = positions[rows] - positions[cols]
        r = vec.norm(dim=1, keepdim=True)
        y = spherical_harmonics(self.lmax, vec / r)
        radial = torch.sin(r * self.freq) / r                       # Bessel-like basis of the edge length
        w = torch.nn.functional.silu(radial @ self.w1) @ self.w2      # per-edge weights
        z = conv(self.embed[species], y.contiguous(), w.contiguous())
        return (z * self.readout).sum()


def train_step(block, positions, species, rows, cols, conv, e_ref, f_ref):
    """Energy, forces (kept differentiable) and the gradients of an energy + force loss."""
    positions = positions.clone().requires_grad_(True)
    energy = block.energy(positions, species, rows, cols, conv)
    forces = -torch.autograd.grad(energy, positions, create_graph=True)[0]
    loss = (energy - e_ref) ** 2 + ((forces - f_ref) ** 2).sum()
    grads = torch.autograd.grad(loss, list(block.parameters()))
    return energy.detach(), forces.detach(), grads


@pytest.mark.parametrize("deterministic", [True, False], ids=["deterministic", "atomic"])
@pytest.mark.parametrize("dtype,tol", [(torch.float64, 1e-9), (torch.float32, 2e-3)], ids=["f64", "f32"])
def test_energy_force_training_step(dtype, tol, deterministic):
    np_dtype = np.float64 if dtype == torch.float64 else np.float32
    problem = problem_by_name("interaction_8", irrep_dtype=np_dtype, weight_dtype=np_dtype)
    rng = np.random.default_rng(5)
    nodes = 40
    pos = rng.uniform(0.0, 2.2, size=(nodes, 3))
    rows, cols, perm = neighbour_graph(pos, cutoff=1.0)
    assert len(rows) > 4 * nodes
    species = torch.from_numpy(rng.integers(0, 3, size=nodes))
    f_ref = torch.from_numpy(rng.normal(size=(nodes, 3)))
    e_ref = torch.tensor(0.3, dtype=torch.float64)

    # oracle: float64 on the CPU
    ref = InteractionBlock(problem, lmax=1)
    r_c, c_c = torch.from_numpy(rows), torch.from_numpy(cols)
    want = train_step(ref, torch.from_numpy(pos), species, r_c, c_c,
                      lambda x, y, w: orc.conv_torch(problem, x, y, w, r_c, c_c), e_ref, f_ref)

    # the library on the GPU
    block = InteractionBlock(problem, lmax=1).to(device="cuda", dtype=dtype)
    conv = oeq.TensorProductConv(problem, torch_op=True, deterministic=deterministic)
    fused_calls = []
    inner = conv._double_backward_impl
    conv._double_backward_impl = lambda *a, **k: (fused_calls.append(1), inner(*a, **k))[1]
    r_g, c_g, p_g = (torch.from_numpy(a).cuda() for a in (rows, cols, perm))
    index = (r_g, c_g, p_g) if deterministic else (r_g, c_g)
    got = train_step(block, torch.from_numpy(pos).to(device="cuda", dtype=dtype), species.cuda(), r_g, c_g,
                     lambda x, y, w: conv.forward(x, y, w, *index), e_ref.to(device="cuda", dtype=dtype),
                     f_ref.to(device="cuda", dtype=dtype))
    conv.check_device_status()
    assert fused_calls, "the second derivatives of the convolution should have taken the fused launches"

    def close(a, b):
        a, b = a.detach().cpu().double(), b.double()
        return float((a - b).abs().max() / max(float(b.abs().max()), 1e-30))

    assert close(got[0], want[0]) < tol
    assert close(got[1], want[1]) < tol
    for g, w in zip(got[2], want[2]):
        assert close(g, w) < tol
