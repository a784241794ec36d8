"""Writes random-init GRACE-3L models in the reference's `kokkos.npz` format.

No GRACE-3L file ships with the reference, so the architecture tables are built here from first principles instead of
being taken from a fixture: every coupling (the equivariant SPBF's `cg_W`, the `cp_l` products) uses Gaunt
coefficients of the real spherical harmonics the engines evaluate (Y_00 = 1, lm = l (l + 1) + m,
libgrace/include/grace/fused_cpu.h:686-798), integrated exactly by quadrature, so a generated model is a rotation
invariant function of the structure.  The keys, shapes and the layer graph are the ones the loader checks
(libgrace/src/model_3l.cpp:36-154 dataflow, :165-464 keys) and the shape class is the one the CPU engine accepts
(libgrace/src/fused_3l.cpp:373-375, 433, 462, 815-822: channels a multiple of 16, three-layer radial MLP with bias on
the hidden layers, element-dependent invariant rho reduces, two-layer energy MLP).

Per layer k (K = A1, A2, A3; X = A1 itself or the reduce of the equivariant SPBF):
    K_2 = cp_l(X, X) -> K_2_red;  K_2a = fc(K_2_red, X);  K_3 = cp_l(K_2a, X) -> K_3_red;
    K_2b = fc(K_2_red, X);  K_4 = cp_l(K_2b, K_2b) -> K_4_red;
    eq{k} = reduce(X, K_2_red, K_3_red, K_4_red) -> eq{k}_norm (message of layer k + 1, k < 3);
    rho{k} = invariant reduce of the same -> rho{k}_norm;  E = MLP(sum_k rho{k}_norm).
"""
from __future__ import annotations

import numpy as np


def _lm_l(lmax):
    return np.array([l for l in range(lmax + 1) for _ in range(2 * l + 1)], dtype=np.int64)


def real_sh(u, lmax):
    """Real spherical harmonics of unit vectors u [n, 3], normalised to Y_00 = 1 (integral of Y^2 over the sphere
    = 4 pi), Condon-Shortley phase, lm = l (l + 1) + m with m > 0 the cosine and m < 0 the sine functions."""
    u = np.asarray(u, dtype=np.float64)
    x, y, z = u[:, 0], u[:, 1], u[:, 2]
    s = np.sqrt(np.maximum(0.0, 1.0 - z * z))
    phi = np.arctan2(y, x)
    P = {}
    for m in range(lmax + 1):
        pmm = np.ones_like(z)
        for k in range(1, m + 1):
            pmm = -pmm * (2 * k - 1) * s
        P[(m, m)] = pmm
        if m + 1 <= lmax:
            P[(m + 1, m)] = z * (2 * m + 1) * pmm
        for l in range(m + 2, lmax + 1):
            P[(l, m)] = ((2 * l - 1) * z * P[(l - 1, m)] - (l + m - 1) * P[(l - 2, m)]) / (l - m)
    Y = np.zeros((u.shape[0], (lmax + 1) ** 2))
    for l in range(lmax + 1):
        for m in range(l + 1):
            ratio = 1.0
            for k in range(l - m + 1, l + m + 1):
                ratio /= k
            nrm = np.sqrt((2 * l + 1) * ratio)
            if m == 0:
                Y[:, l * (l + 1)] = nrm * P[(l, 0)]
            else:
                f = np.sqrt(2.0) * (-1) ** m * nrm * P[(l, m)]
                Y[:, l * (l + 1) + m] = f * np.cos(m * phi)
                Y[:, l * (l + 1) - m] = f * np.sin(m * phi)
    return Y


def gaunt(lmax):
    """G[a, b, c] = 1 / (4 pi) integral Y_a Y_b Y_c over the sphere for all lm up to lmax: Gauss-Legendre in cos(theta),
    uniform in phi, exact for the polynomial degree 3 lmax."""
    nz, nphi = 2 * lmax + 4, 4 * lmax + 4
    zs, wz = np.polynomial.legendre.leggauss(nz)
    ph = 2.0 * np.pi * np.arange(nphi) / nphi
    zz, pp = np.meshgrid(zs, ph, indexing="ij")
    st = np.sqrt(1.0 - zz * zz)
    u = np.stack([st * np.cos(pp), st * np.sin(pp), zz], axis=-1).reshape(-1, 3)
    w = np.repeat(wz, nphi) / (2.0 * nphi)
    Y = real_sh(u, lmax)
    G = np.einsum("q,qa,qb,qc->abc", w, Y, Y, Y)
    G[np.abs(G) < 1e-12] = 0.0
    return G


def _paths(lmax, Lmax, ordered):
    out = []
    for l1 in range(lmax + 1):
        for l2 in (range(lmax + 1) if ordered else range(l1, lmax + 1)):
            for L in range(abs(l1 - l2), min(l1 + l2, Lmax) + 1):
                if (l1 + l2 + L) % 2 == 0:
                    out.append((l1, l2, L))
    return out


def _couplings(G, lmax, Lmax, ordered):
    """Terms (left lm, right lm, output function, coefficient) of all paths (l1, l2 -> L); output function f of path p
    and M is consecutive; per path the coefficients are scaled to sum of squares 2 L + 1."""
    left, right, out, cg, f_l, f_path, f_lm = [], [], [], [], [], [], []
    lml = _lm_l(lmax)
    for p, (l1, l2, L) in enumerate(_paths(lmax, Lmax, ordered)):
        a = np.nonzero(lml == l1)[0]
        b = np.nonzero(lml == l2)[0]
        block = G[np.ix_(a, b, np.arange(L * L, (L + 1) ** 2))]
        scale = np.sqrt((2 * L + 1) / np.sum(block * block))
        f0 = len(f_l)
        for M in range(2 * L + 1):
            f_l.append(L)
            f_path.append(p)
            f_lm.append(L * L + M)
        ia, ib, ic = np.nonzero(block)
        for q in range(len(ia)):
            left.append(a[ia[q]])
            right.append(b[ib[q]])
            out.append(f0 + ic[q])
            cg.append(block[ia[q], ib[q], ic[q]] * scale)
    i64 = lambda v: np.array(v, dtype=np.int64)
    return dict(left=i64(left), right=i64(right), out=i64(out), cg=np.array(cg), f_l=i64(f_l), f_path=i64(f_path),
                f_lm=i64(f_lm), npaths=len(_paths(lmax, Lmax, ordered)))


def _names(v):
    return np.array([s.encode() for s in v])


def _i(v):
    return np.array([v], dtype=np.int64)


def _f(v):
    return np.array([v], dtype=np.float64)


def write_model_3l(path, elements=("Al", "Ni"), lmax=2, channels=(16, 16, 16), rho_width=16, embedding=8, nradbase=8,
                   radial_hidden=32, energy_hidden=32, rcut=5.0, p=5, avg_neigh=30.0, seed=0):
    """A GRACE-3L `kokkos.npz` with weights W ~ N(0, 1) next to `*_norm = 1 / sqrt(fan_in)`.  `channels` = n_rad_max of
    A1, A2, A3 (multiples of 16); the messages eq1_norm / eq2_norm carry all (lmax + 1)^2 functions with the channels
    of the layer they feed."""
    rng = np.random.default_rng(seed)
    ne, nl, nlm = len(elements), lmax + 1, (lmax + 1) ** 2
    lml = _lm_l(lmax)
    G = gaunt(lmax)
    sym = _couplings(G, lmax, lmax, ordered=False)     # X x X and FB x FB
    full = _couplings(G, lmax, lmax, ordered=True)     # FA x X and Y x message
    o = {}

    def w(key, shape, fan_in, norm_key=None):
        o[key] = rng.standard_normal(shape)
        if norm_key:
            o[norm_key] = _f(1.0 / np.sqrt(fan_in))

    o["grace_model_kind"] = _names(["GRACE-3L"])
    o["grace_format_version"] = _i(1)
    o["n_elements"] = _i(ne)
    o["embedding_size"] = _i(embedding)
    o["nradbase"] = _i(nradbase)
    o["rcut"] = _f(rcut)
    o["has_bond_specific_cutoff"] = _i(0)
    o["bond_cutoff_map"] = np.full((ne, ne), float(rcut))
    o["chem_embedding"] = rng.standard_normal((ne, embedding))
    o["shift_values"] = 0.1 * rng.standard_normal(ne)
    o["output_scale"] = _f(1.0)
    o["element_names"] = _names(elements)

    def mlp(prefix, widths, bias):
        o[prefix + "_n_layers"] = _i(len(widths) - 1)
        for q in range(len(widths) - 1):
            w(f"{prefix}_W{q}", (widths[q], widths[q + 1]), widths[q], f"{prefix}_norm{q}")
            if bias and q < len(widths) - 2:
                o[f"{prefix}_b{q}"] = 0.1 * rng.standard_normal(widths[q + 1])

    def reduce_instr(name, src, n_in, n_out, collect, tile, total, w_shape, elem):
        o[f"{name}_n_in_{src}"] = _i(n_in)
        o[f"{name}_w_shape_{src}"] = _i(w_shape)
        shape = (ne, n_out, n_in, w_shape) if elem else (n_out, n_in, w_shape)
        per_out = np.maximum(1, np.bincount(total, minlength=int(total.max()) + 1)).mean()
        w(f"{name}_reduce_{src}_W", shape, n_in * per_out, f"{name}_reduce_{src}_norm")
        o[f"{name}_collect_ind_{src}"] = collect.astype(np.int64)
        o[f"{name}_w_l_tile_{src}"] = tile.astype(np.int64)
        o[f"{name}_total_sum_ind_{src}"] = total.astype(np.int64).reshape(-1, 1)

    def reduce(name, sources, n_out, n_funcs, only_invar=False, elem=False):
        o[f"{name}_n_out"] = _i(n_out)
        o[f"{name}_n_funcs"] = _i(n_funcs)
        o[f"{name}_only_invar"] = _i(int(only_invar))
        o[f"{name}_is_central_atom_type_dependent"] = _i(int(elem))
        o[f"{name}_instruction_names"] = _names([s[0] for s in sources])
        for src, n_in, collect, tile, total, w_shape in sources:
            reduce_instr(name, src, n_in, n_out, collect, tile, total, w_shape, elem)
        o[f"{name}_norm_map"] = np.full(1 if only_invar else n_funcs, 1.0 / np.sqrt(len(sources)))

    def cpl(name, tab, n_left, n_right, rank):
        o[f"{name}_rank"] = _i(rank)
        o[f"{name}_nfunc"] = _i(len(tab["f_l"]))
        o[f"{name}_n_left"] = _i(n_left)
        o[f"{name}_n_right"] = _i(n_right)
        o[f"{name}_n_groups_left"] = _i(nl)
        o[f"{name}_n_groups_right"] = _i(nl)
        w(f"{name}_U", (nl, rank, n_left), n_left, f"{name}_norm_u")
        w(f"{name}_V", (nl, rank, n_right), n_right, f"{name}_norm_v")
        o[f"{name}_cg"] = tab["cg"].copy()
        o[f"{name}_group_left"] = lml.copy()
        o[f"{name}_group_right"] = lml.copy()
        o[f"{name}_left_ind"] = tab["left"].copy()
        o[f"{name}_right_ind"] = tab["right"].copy()
        o[f"{name}_m_sum_ind"] = tab["out"].copy()
        o[f"{name}_out_l"] = tab["f_l"].copy()

    def prod_reduce(name, tab, rank, n_out):      # reduce of a cp_l product: one weight tile per path
        nf = len(tab["f_l"])
        reduce(name + "_red", [(name, rank, np.arange(nf), tab["f_path"], tab["f_lm"], tab["npaths"])], n_out, nlm)

    def fc(name, n_out, n_in_right):
        pre = "fc_" + name
        o[pre + "_n_out"] = _i(n_out)
        o[pre + "_left_coefs"] = _i(0)
        w(pre + "_w_right", (n_out, n_in_right, nl), n_in_right, pre + "_norm_right")
        o[pre + "_w_tile_left"] = lml.copy()
        o[pre + "_w_tile_right"] = lml.copy()
        o[pre + "_collect_from"] = np.arange(nlm, dtype=np.int64)
        o[pre + "_collect_to"] = np.arange(nlm, dtype=np.int64)
        o[pre + "_norm_out_factor"] = np.full((nlm, 1, 1), 1.0 / np.sqrt(2.0))

    spbf, prods, reduces, fcs, eqnorms, rmsnorms = [], [], [], [], [], []
    for k in (1, 2, 3):
        K, C = f"A{k}", channels[k - 1]
        if C % 16:
            raise ValueError("channels must be multiples of 16")
        spbf.append(K)
        o[K + "_equivariant"] = _i(int(k > 1))
        o[K + "_n_rad_max"] = _i(C)
        o[K + "_n_rad_basis"] = _i(nradbase)
        o[K + "_lmax"] = _i(lmax)
        o[K + "_Lmax"] = _i(lmax)
        o[K + "_p"] = _i(p)
        o[K + "_rcut"] = _f(rcut)
        o[K + "_inv_avg_n_neigh"] = _f(1.0 / avg_neigh)
        o[K + "_l_tile"] = lml.copy()
        mlp(K + "_mlp", [nradbase + 2 * embedding, radial_hidden, radial_hidden, C * nl], bias=True)
        X = K
        if k == 1:
            w(K + "_lin_transform_W", (embedding, C), embedding, K + "_lin_transform_norm")
        else:
            nf = len(full["f_l"])
            o[K + "_nfunc"] = _i(nf)
            o[K + "_n_lm_ind"] = _i(nlm)
            w(K + "_chem_linear_W", (embedding, C), embedding, K + "_chem_linear_norm")
            o[K + "_chem_l0_mask"] = (np.arange(nlm) == 0).astype(np.float64)
            cgw = np.zeros((nlm * nlm, nf))
            cgw[full["left"] * nlm + full["right"], full["out"]] = full["cg"]
            o[K + "_cg_W"] = cgw
            reduce(K + "_red", [(K, C, np.arange(nf), full["f_path"], full["f_lm"], full["npaths"])], C, nlm)
            reduces.append(K + "_red")
            X = K + "_red"
        cpl(K + "_2", sym, C, C, C)
        prods.append(K + "_2")
        prod_reduce(K + "_2", sym, C, C)
        reduces.append(K + "_2_red")
        fc(K + "_2a", C, C)
        cpl(K + "_3", full, C, C, C)
        prods.append(K + "_3")
        prod_reduce(K + "_3", full, C, C)
        reduces.append(K + "_3_red")
        fc(K + "_2b", C, C)
        cpl(K + "_4", sym, C, C, C)
        prods.append(K + "_4")
        prod_reduce(K + "_4", sym, C, C)
        reduces.append(K + "_4_red")
        fcs += [K + "_2a", K + "_2b"]
        collect = [X, K + "_2_red", K + "_3_red", K + "_4_red"]
        if k < 3:
            Cn = channels[k]
            reduce(f"eq{k}", [(s, C, np.arange(nlm), lml, np.arange(nlm), nl) for s in collect], Cn, nlm)
            reduces.append(f"eq{k}")
            e = f"eq{k}_norm"
            eqnorms.append(e)
            o[e + "_affine_weight"] = 1.0 + 0.1 * rng.standard_normal((nl, Cn))
            o[e + "_degree_weights"] = 1.0 / ((2.0 * lml + 1.0) * nl)
            o[e + "_l0_mask"] = (np.arange(nlm) == 0).astype(np.float64)
            o[e + "_expand_index"] = lml.copy()
            o[e + "_eps"] = _f(1e-8)
            o[e + "_center_l0"] = _i(1)
        z = np.zeros(1, dtype=np.int64)
        reduce(f"rho{k}", [(s, C, z, z, z, 1) for s in collect], rho_width, 1, only_invar=True, elem=True)
        reduces.append(f"rho{k}")
        r = f"rho{k}_norm"
        rmsnorms.append(r)
        o[r + "_scale"] = 1.0 + 0.1 * rng.standard_normal(rho_width - 1)
        o[r + "_type"] = _i(1)
        o[r + "_n_out"] = _i(rho_width)
    o["spbf_names"] = _names(spbf)
    o["prod_names"] = _names(prods)
    o["reduce_names"] = _names(reduces)
    o["fc_names"] = _names(fcs)
    o["eqnorm_names"] = _names(eqnorms)
    o["rmsnorm_names"] = _names(rmsnorms)
    o["out1_origins"] = _names(rmsnorms)
    o["energy_mlp_origin_n_out"] = _i(rho_width)
    o["energy_mlp_n_origins"] = _i(3)
    mlp("energy_mlp", [rho_width - 1, energy_hidden, 1], bias=False)
    o["energy_mlp_activation"] = _i(0)
    np.savez(path, **o)
    return path
