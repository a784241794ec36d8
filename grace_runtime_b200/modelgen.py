"""Writes random-init GRACE-1L / GRACE-2L models in the reference's `kokkos.npz` format.

The file layout follows what the reference loaders read (libgrace/src/model_1l.cpp:18-273,
libgrace/src/model_2l.cpp:28-400): weights W ~ N(0, 1) stored as float64 next to a scalar `*_norm = 1/sqrt(fan_in)`
(the convention of every fixture of the reference test tree), uncompressed npz, C order.  The architecture tables
(function indices, Clebsch-Gordan coefficients, tile maps) come from `data/topology_*.npz`.

`CONFIGS` holds the benchmark architectures.  The radial basis is the format's Chebyshev x envelope basis
(libgrace/include/grace/radial_x.h:11-26): the file format has no key for another one.
"""
from __future__ import annotations

import os

import numpy as np

_DATA = os.path.join(os.path.dirname(os.path.abspath(__file__)), "data")

ELEMENTS = ("H He Li Be B C N O F Ne Na Mg Al Si P S Cl Ar K Ca Sc Ti V Cr Mn Fe Co Ni Cu Zn Ga Ge As Se Br Kr Rb Sr "
            "Y Zr Nb Mo Tc Ru Rh Pd Ag Cd In Sn Sb Te I Xe Cs Ba La Ce Pr Nd Pm Sm Eu Gd Tb Dy Ho Er Tm Yb Lu Hf Ta W "
            "Re Os Ir Pt Au Hg Tl Pb Bi Po At Rn Fr Ra Ac").split()
assert len(ELEMENTS) == 89


def _topology(layers, lmax, max_order):
    names = {(1, 4): "topology_1l_lmax4", (1, 3): "topology_1l_lmax3_o3", (1, 2): "topology_1l_lmax2",
             (2, 3): "topology_2l_lmax3_o3", (2, 2): "topology_2l_lmax2"}
    if (layers, lmax) not in names:
        raise ValueError(f"no architecture tables for a {layers}L model with lmax {lmax}")
    z = np.load(os.path.join(_DATA, names[(layers, lmax)] + ".npz"))
    t = {k: z[k] for k in z.files}
    has4 = "prod_AAAA_n_cg_terms" in t
    if max_order == 4 and not has4:
        raise ValueError(f"the lmax {lmax} tables have no order-4 stage")
    if max_order == 3 and has4:      # an order-3 file has none of the AAAA / BBBB / fc_AA2 / fc_BB2 arrays
        drop = [k for k in t if "AAAA" in k or "BBBB" in k or k.startswith(("fc_AA2_", "fc_BB2_"))]
        for k in drop:
            del t[k]
        for k in [k for k in t if k.endswith("_instruction_names")]:
            t[k] = np.array([x for x in t[k] if x not in (b"AAAA", b"BBBB")], dtype=t[k].dtype)
    return t


def _i(v):
    return np.array([v], dtype=np.int64)


def _f(v):
    return np.array([v], dtype=np.float64)


class _Writer:
    def __init__(self, topo, rng):
        self.t, self.rng, self.out = topo, rng, dict(topo)

    def w(self, key, shape, fan_in, norm_key=None, scalar_shape=(1,)):
        self.out[key] = self.rng.standard_normal(shape)
        if norm_key:
            self.out[norm_key] = np.full(scalar_shape, 1.0 / np.sqrt(fan_in))

    def mlp(self, prefix, widths):
        for i in range(len(widths) - 1):
            self.w(f"{prefix}_W{i}", (widths[i], widths[i + 1]), widths[i], f"{prefix}_norm{i}")
        self.out[f"{prefix}_n_layers"] = _i(len(widths) - 1)

    def fc(self, name, n_out, n_in_left, n_in_right):
        if f"{name}_w_tile_left" not in self.t:
            return
        tl = int(self.t[f"{name}_w_tile_left"].max()) + 1
        tr = int(self.t[f"{name}_w_tile_right"].max()) + 1
        self.w(f"{name}_w_left", (n_out, n_in_left, tl), n_in_left, f"{name}_norm_left", ())
        self.w(f"{name}_w_right", (n_out, n_in_right, tr), n_in_right, f"{name}_norm_right", ())
        self.out[f"{name}_n_out"] = _i(n_out)

    def reduce(self, prefix, src, lead, n_out, n_in):
        if f"{prefix}_collect_ind_{src}" not in self.t:
            return
        ws = int(self.t[f"{prefix}_w_shape_{src}"].reshape(-1)[0])
        self.w(f"{prefix}_reduce_{src}_W", tuple(lead) + (n_out, n_in, ws), n_in, f"{prefix}_reduce_{src}_norm", ())
        self.out[f"{prefix}_n_in_{src}"] = _i(n_in)


def write_model(path, layers=1, lmax=4, max_order=3, elements=("W",), embedding=16, nradbase=8, rcut=6.0, p=5,
                hidden=(64, 64), c1=32, fc1=None, cr=16, c2=64, i1_out=12, rho_n_out=9, energy_hidden=(64,),
                avg_neigh=58.0, seed=0, shift_scale=0.0, bond_cutoffs=None):
    """Write a seeded random-init model.  c1: layer-1 radial channels (1L: nradmax); fc1: 1L FC width (default c1);
    cr / c2: 2L message channels / layer-2 FC width; energy_hidden=() gives a linear readout."""
    rng = np.random.default_rng(seed)
    t = _topology(layers, lmax, max_order)
    W = _Writer(t, rng)
    o = W.out
    nel, nl = len(elements), lmax + 1
    fc1 = c1 if (fc1 is None or layers == 2) else fc1
    o["grace_model_kind"] = np.array([f"GRACE-{layers}L".encode()], dtype="|S8")
    o["grace_format_version"] = _i(1)
    o["n_elements"] = _i(nel)
    o["element_names"] = np.array([e.encode() for e in elements], dtype="|S2")
    o["embedding_size"] = _i(embedding)
    o["chem_embedding_size"] = _i(embedding)
    o["nradbase"] = _i(nradbase)
    o["rcut"] = _f(rcut)
    o["radial_basis_p"] = _i(p)
    o["lmax"] = _i(lmax)
    o["has_bond_specific_cutoff"] = _i(0 if bond_cutoffs is None else 1)
    if bond_cutoffs is not None:
        o["bond_cutoff_map"] = np.asarray(bond_cutoffs, dtype=np.float64).reshape(nel, nel)
    o["chem_embedding"] = rng.standard_normal((nel, embedding))
    W.w("A_lin_transform_W", (embedding, c1), embedding, "A_lin_transform_norm")
    o["A_inv_avg_n_neigh"] = np.array(1.0 / avg_neigh)
    if layers == 1:
        o["nradmax"] = _i(c1)
        W.mlp("mlp_rad", (nradbase,) + tuple(hidden) + (c1 * nl,))
        o["mlp_rad_n_rad_max"] = _i(c1)
        W.fc("fc_A1", fc1, c1, c1)
        W.fc("fc_AA1", fc1, fc1, c1)
        W.fc("fc_AA2", fc1, fc1, c1)
        W.reduce("rho", "A", (nel,), rho_n_out, c1)
        for s in ("AA", "AAA", "AAAA"):
            W.reduce("rho", s, (nel,), rho_n_out, fc1)
    else:
        W.mlp("mlp_rad_R", (nradbase,) + tuple(hidden) + (c1 * nl,))
        o["mlp_rad_R_n_rad_max"] = _i(c1)
        W.mlp("mlp_rad_R1", (nradbase,) + tuple(hidden) + (cr * nl,))
        o["mlp_rad_R1_n_rad_max"] = _i(cr)
        W.w("B0_lin_transform_W", (embedding, cr), embedding, "B0_lin_transform_norm")
        o["B0_inv_avg_n_neigh"] = np.array(1.0 / avg_neigh)
        o["YI_inv_avg_n_neigh"] = np.array(1.0 / avg_neigh)
        o["YI_n_rad_max"] = _i(cr)
        for name in ("fc_A1", "fc_AA1", "fc_AA2"):
            W.fc(name, c1, c1, c1)
        for name in ("fc_B1", "fc_BB1", "fc_BB2"):
            W.fc(name, c2, c2, c2)
        for s in ("A", "AA", "AAA", "AAAA"):
            W.reduce("I1", s, (nel,), i1_out, c1)
            W.reduce("rho", s, (nel,), rho_n_out, c1)
        o["I1_n_out"] = _i(i1_out)
        W.reduce("I", "I1", (), cr, i1_out)
        o["I_n_out"] = _i(cr)
        W.reduce("B", "YI", (), c2, cr)
        W.reduce("B", "B0", (), c2, cr)
        o["B_n_out"] = _i(c2)
        for s in ("B", "BB", "BBB", "BBBB"):
            W.reduce("I2", s, (nel,), rho_n_out, c2)
        o["I2_n_out"] = _i(rho_n_out)
        o["I_nl_LN_scale"] = 1.0 + 0.1 * rng.standard_normal(rho_n_out - 1)
        o["I_nl_LN_n_out"] = _i(rho_n_out)
        o["I_nl_LN_type"] = _i(1)
        o["I_0_LN_scale"] = 1.0 + 0.1 * rng.standard_normal(rho_n_out)
        o["I_0_LN_n_out"] = _i(rho_n_out)
        o["I_0_LN_type"] = _i(0)
    o["rho_n_out"] = _i(rho_n_out)
    for k in [k for k in o if k.endswith("_number_of_atom_types")]:
        o[k] = _i(nel)
    W.mlp("energy_mlp", (rho_n_out - 1,) + tuple(energy_hidden) + (1,))
    o["shift_values"] = shift_scale * rng.standard_normal(nel)
    os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
    with open(path, "wb") as f:
        np.savez(f, **o)
    return path


def _subset(seed, k):
    """k of the 89 elements, seeded."""
    return [ELEMENTS[i] for i in sorted(np.random.default_rng(seed).choice(89, size=k, replace=False))]


# The benchmark architectures.  `full=True` writes the 89-element tables; the parity-test variants keep the species in
# use (the per-element tables are the only arrays that grow with the element count).
CONFIGS = {
    # GRACE-1L: lmax 4, 32 radial channels, MLP 8 -> 64 -> 64 -> 32 x 5, 16-dim embedding, body order 4, linear readout
    "1l": dict(layers=1, lmax=4, max_order=3, embedding=16, nradbase=8, rcut=6.0, hidden=(64, 64), c1=32,
               rho_n_out=9, energy_hidden=(), avg_neigh=58.0),
    # GRACE-2L: lmax 3, layer 1: 32 radial channels, rank 3; message 4 functions x 16 channels = 64 floats per atom;
    # layer 2: radial MLP 8 -> 64 -> 64 -> 16 x 4, FC width 64, scalar readout through a 64-wide energy MLP
    "2l": dict(layers=2, lmax=3, max_order=3, embedding=16, nradbase=8, rcut=6.0, hidden=(64, 64), c1=32, cr=16,
               c2=64, i1_out=12, rho_n_out=9, energy_hidden=(64,), avg_neigh=78.0),
}


def write_config_model(path, config, elements, seed=0):
    return write_model(path, elements=tuple(elements), seed=seed, **CONFIGS[config])


def uq_basis_width(z):
    """Rows of the UQ projection matrix of a model file (dict of arrays): the collected inputs of its scalar reduces,
    blocks in the order of the reference (libgrace/src/model_1l.cpp:306-316, libgrace/src/model_2l.cpp:520-535)."""
    blocks = [("I2", ("B", "BB", "BBB", "BBBB")), ("rho", ("A", "AA", "AAA", "AAAA"))]
    if "I2_reduce_B_W" not in z:
        blocks = blocks[1:]
    width = 0
    for prefix, sources in blocks:
        for s in sources:
            if f"{prefix}_reduce_{s}_W" not in z:
                raise ValueError("a UQ head needs a max_order 4 model (libgrace/src/model_1l.cpp:278)")
            width += z[f"{prefix}_reduce_{s}_W"].shape[-2] * len(np.asarray(z[f"{prefix}_collect_ind_{s}"]).reshape(-1))
    return width, len(blocks)


def add_uq_head(src, dst, seed=0, rp_dim=32, max_clusters=3):
    """Copies the model file `src` to `dst` with a seeded random UQ head of schema 6 (keys and checks:
    libgrace/src/uq_head.cpp:12-78): projection matrix, Gaussian-mixture centroids, precision matrices and
    thresholds for every element.  The published models carry fitted heads; a random one has the same arithmetic."""
    z0 = np.load(src)
    z = {k: z0[k] for k in z0.files}
    rng = np.random.default_rng(seed)
    d_basis, nblocks = uq_basis_width(z)
    nel = int(np.asarray(z["n_elements"]).reshape(-1)[0]) if "n_elements" in z else 89
    D = rp_dim + 1 + nblocks
    z["uq_schema_version"] = _i(6)
    z["uq_n_elements"] = _i(nel)
    z["uq_max_clusters"] = _i(max_clusters)
    z["uq_rp_dim"] = _i(rp_dim)
    z["uq_feature_dim"] = _i(D)
    z["uq_rp_normalize"] = _i(1)
    z["uq_rp_add_density_channel"] = _i(1)
    z["uq_rp_density_scale"] = _f(1.0)
    z["uq_feature_transform"] = _i(0)
    z["uq_rp_matrix"] = rng.standard_normal((d_basis, rp_dim))
    z["uq_centroids"] = rng.standard_normal((nel, max_clusters, D))
    m = rng.standard_normal((nel, max_clusters, D, D)) / np.sqrt(D)
    z["uq_inv_cov"] = m @ m.transpose(0, 1, 3, 2) + np.eye(D)
    z["uq_n_clusters"] = rng.integers(1, max_clusters + 1, size=nel).astype(np.int64)
    z["uq_interp_thresholds"] = 1.0 + 2.0 * rng.random((nel, max_clusters))
    os.makedirs(os.path.dirname(os.path.abspath(dst)), exist_ok=True)
    with open(dst, "wb") as f:
        np.savez(f, **z)
    return dst
