"""TEST INFRASTRUCTURE: numpy fp64 restatement of the GRACE-3L forward pass (per-atom energies) of the reference's CPU
engine.  Only tests/, smoke and bench legs may import this; the library never does.

Follows libgrace/src/fused_3l.cpp: radial functions by cubic Hermite tables of the pair-dependent MLP (:307-351,
:439-533), scalar and equivariant SPBF (:1276-1310, bond vectors :1055-1081), the chain cp_l -> reduce -> fc of a layer
(:992-1009 with :904-975), EquivariantRMSNorm and RMSNorm (libgrace/include/grace/fused_3l_cpu.h:346-370, 416-425),
readout (:1334-1357).  Pinned against the compiled reference on generated model files (tests/test_model3l.py): the
reference tree has no GRACE-3L model, so there are no golden vectors of its own for this path - parity of GRACE-3L is
"unpinned" beyond this oracle-vs-reference check.
"""
from __future__ import annotations

import numpy as np

from .grace_oracle import Npz, neighbor_list, sph_harm


def _silu(s):
    sg = 1.0 / (1.0 + np.exp(-s))
    return s * sg, sg * (1.0 + s * (1.0 - sg))


class Grace3LOracle:
    def __init__(self, path, spline_n=1024):
        z = self.z = Npz(path)
        self.N = spline_n
        self.ne = z.is_("n_elements")
        self.emb = z.is_("embedding_size", 64)
        self.nrb = z.is_("nradbase", 10)
        self.lmax = z.is_("A1_lmax", 4)
        self.nl, self.nlm = self.lmax + 1, (self.lmax + 1) ** 2
        self.rcut = z.fs("rcut", 6.0)
        self.chem = z.f("chem_embedding").reshape(self.ne, self.emb)
        self.shift = z.f("shift_values")
        self.oscale = z.fs("output_scale", 1.0)
        self.elements = z.names("element_names")
        self.cutmap = np.full((self.ne, self.ne), self.rcut)
        if z.is_("has_bond_specific_cutoff", 0):
            self.cutmap = z.f("bond_cutoff_map").reshape(self.ne, self.ne)
        self._tables = {}

    # ---- radial ------------------------------------------------------------------------------------------------
    def _mlp(self, K, x, zi, zj):
        """value and d/dx of the radial MLP of layer K at the points x (fp64, forward mode)."""
        z = self.z
        t = 2.0 * x - 1.0
        T, dT = [np.ones_like(t), t], [np.zeros_like(t), 2.0 * np.ones_like(t)]
        for _ in range(self.nrb):
            T.append(2.0 * t * T[-1] - T[-2])
            dT.append(2.0 * (2.0 * T[-2] + t * dT[-1]) - dT[-2])
        h = np.concatenate([np.stack(T[1:self.nrb + 1], 1), np.tile(zi, (len(x), 1)), np.tile(zj, (len(x), 1))], 1)
        dh = np.concatenate([np.stack(dT[1:self.nrb + 1], 1), np.zeros((len(x), 2 * self.emb))], 1)
        nlay = z.is_(K + "_mlp_n_layers")
        for q in range(nlay):
            W, nrm = z.f(f"{K}_mlp_W{q}"), z.fs(f"{K}_mlp_norm{q}", 1.0)
            s, ds = (h @ W) * nrm, (dh @ W) * nrm
            if q < nlay - 1:
                if z.has(f"{K}_mlp_b{q}"):
                    s = s + nrm * z.f(f"{K}_mlp_b{q}")
                act, dact = _silu(s)
                s, ds = act, dact * ds
            h, dh = s, ds
        return h, dh

    def _table(self, k, mui, muj):
        """Hermite coefficients [N][4][nl][C] of layer k (0-based) for the element pair (centre, neighbour)."""
        key = (k, mui, muj)
        if key in self._tables:
            return self._tables[key]
        z, K, N = self.z, f"A{k + 1}", self.N
        C, p = z.is_(K + "_n_rad_max"), z.is_(K + "_p", 5)
        x = np.arange(N + 1) / N
        out, dout = self._mlp(K, x, self.chem[mui], self.chem[muj])
        xp = x ** p
        env = 1.0 - 0.5 * (p + 1) * (p + 2) * xp + p * (p + 2) * xp * x - 0.5 * p * (p + 1) * xp * x * x
        denv = 0.5 * p * (p + 1) * (p + 2) * (-x ** (p - 1) + 2.0 * xp - xp * x)
        fac = np.full(C, z.fs(K + "_inv_avg_n_neigh", 1.0))
        if k == 0:
            fac = fac * (self.chem[muj] @ z.f(K + "_lin_transform_W").reshape(self.emb, C)) * z.fs(K + "_lin_transform_norm", 1.0)
        # MLP output o = c (lmax + 1) + l  ->  [q][l][c]
        f = (out * env[:, None]).reshape(N + 1, C, self.nl).transpose(0, 2, 1) * fac
        d = ((dout * env[:, None] + out * denv[:, None]) / N).reshape(N + 1, C, self.nl).transpose(0, 2, 1) * fac
        f0, f1, d0, d1 = f[:-1], f[1:], d[:-1], d[1:]
        tab = np.stack([f0, d0, -3.0 * f0 - 2.0 * d0 + 3.0 * f1 - d1, 2.0 * f0 + d0 - 2.0 * f1 + d1], 1)
        tab = tab.astype(np.float32).astype(np.float64)       # the engine keeps the tables in fp32
        self._tables[key] = tab
        return tab

    def _radial(self, k, mui, muj, x):
        tab = self._table(k, mui, muj)
        s = x * self.N
        q = min(max(int(s), 0), self.N - 1)
        t = s - q
        c = tab[q]
        return c[0] + t * (c[1] + t * (c[2] + t * c[3]))      # [nl][C]

    # ---- dense operators on [function][channel] tensors of one atom -------------------------------------------------
    def _reduce(self, name, T, mu):
        z = self.z
        n_out = z.is_(name + "_n_out")
        invar, elem = z.is_(name + "_only_invar", 0), z.is_(name + "_is_central_atom_type_dependent", 0)
        nfo = 1 if invar else z.is_(name + "_n_funcs")
        out = np.zeros((nfo, n_out))
        for src in z.names(name + "_instruction_names"):
            W = z.f(f"{name}_reduce_{src}_W") * z.fs(f"{name}_reduce_{src}_norm", 1.0)
            if elem:
                W = W[mu]                                      # [n_out][n_in][tiles]
            ci, ti = z.i(f"{name}_collect_ind_{src}").reshape(-1), z.i(f"{name}_w_l_tile_{src}").reshape(-1)
            to = z.i(f"{name}_total_sum_ind_{src}").reshape(-1)
            X = T[src]
            for c in range(len(ci)):
                out[0 if invar else to[c]] += W[:, :, ti[c]] @ X[ci[c]]
        if z.has(name + "_norm_map"):
            out *= z.f(name + "_norm_map").reshape(-1, 1)
        return out

    def _cpl(self, name, L, R):
        z = self.z
        U, V = z.f(name + "_U") * z.fs(name + "_norm_u", 1.0), z.f(name + "_V") * z.fs(name + "_norm_v", 1.0)
        gl, gr = z.i(name + "_group_left").reshape(-1), z.i(name + "_group_right").reshape(-1)
        Lp = np.stack([U[gl[w]] @ L[w] for w in range(len(gl))])
        Rp = np.stack([V[gr[w]] @ R[w] for w in range(len(gr))])
        out = np.zeros((z.is_(name + "_nfunc"), U.shape[1]))
        li, ri, mi = z.i(name + "_left_ind").reshape(-1), z.i(name + "_right_ind").reshape(-1), z.i(name + "_m_sum_ind").reshape(-1)
        np.add.at(out, mi, z.f(name + "_cg").reshape(-1, 1) * Lp[li] * Rp[ri])
        return out

    def _fc(self, name, left, right):
        z, p = self.z, "fc_" + name
        W = z.f(p + "_w_right") * z.fs(p + "_norm_right", 1.0)      # [n_out][n_in][tiles]
        out = left.copy()
        cf, ct, tt = z.i(p + "_collect_from").reshape(-1), z.i(p + "_collect_to").reshape(-1), z.i(p + "_w_tile_right").reshape(-1)
        for q in range(len(cf)):
            out[ct[q]] += W[:, :, tt[q]] @ right[cf[q]]
        return out * z.f(p + "_norm_out_factor").reshape(-1, 1)

    def _eqnorm(self, name, x):
        z = self.z
        C = x.shape[1]
        mask, dw = z.f(name + "_l0_mask").reshape(-1), z.f(name + "_degree_weights").reshape(-1)
        xc = x.copy()
        if z.is_(name + "_center_l0", 1):
            xc -= (mask * x.mean(1))[:, None]
        r = 1.0 / np.sqrt((dw[:, None] * xc * xc).sum() / C + z.fs(name + "_eps", 1e-8))
        aff = z.f(name + "_affine_weight")[z.i(name + "_expand_index").reshape(-1)]
        return xc * r * aff

    def _rmsnorm(self, name, x):
        z = self.z
        sc = z.f(name + "_scale").reshape(-1)
        n0 = z.is_(name + "_type", 0)
        y = x.copy()
        r = 1.0 / np.sqrt((x[n0:] ** 2).mean() + 1e-10)
        y[n0:] = x[n0:] * r * sc
        return y

    def _chain(self, k, T, X, mu):
        """T[X] holds the layer's lm features; returns (message or None, normalised density)."""
        K, ks = f"A{k + 1}", str(k + 1)
        T[K + "_2"] = self._cpl(K + "_2", T[X], T[X])
        T[K + "_2_red"] = self._reduce(K + "_2_red", T, mu)
        T[K + "_2a"] = self._fc(K + "_2a", T[K + "_2_red"], T[X])
        T[K + "_3"] = self._cpl(K + "_3", T[K + "_2a"], T[X])
        T[K + "_3_red"] = self._reduce(K + "_3_red", T, mu)
        T[K + "_2b"] = self._fc(K + "_2b", T[K + "_2_red"], T[X])
        T[K + "_4"] = self._cpl(K + "_4", T[K + "_2b"], T[K + "_2b"])
        T[K + "_4_red"] = self._reduce(K + "_4_red", T, mu)
        msg = self._eqnorm(f"eq{ks}_norm", self._reduce("eq" + ks, T, mu)) if k < 2 else None
        rho = self._rmsnorm(f"rho{ks}_norm", self._reduce("rho" + ks, T, mu)[0])
        return msg, rho

    # ---- evaluation --------------------------------------------------------------------------------------------
    def compute(self, species, types, pos, cell, pbc):
        """Per-atom energies and their sum (forward pass only)."""
        z = self.z
        mus = np.array([self.elements.index(s) for s in species])
        mu = mus[np.asarray(types) - 1]
        n = len(mu)
        pos, cell = np.asarray(pos, dtype=np.float64), np.asarray(cell, dtype=np.float64).reshape(3, 3)
        bi, bj, S = neighbor_list(pos, cell, pbc, float(self.cutmap[np.ix_(mus, mus)].max()))
        d = pos[bj] + S @ cell - pos[bi]
        r = np.linalg.norm(d, axis=1)
        rc = self.cutmap[mu[bi], mu[bj]]
        keep = r < rc
        bi, bj, d, r, rc = bi[keep], bj[keep], d[keep], r[keep], rc[keep]
        Y = sph_harm(d / r[:, None], self.lmax)[0]
        l_of = z.i("A1_l_tile").reshape(-1)
        msg_prev = None
        rho_sum = np.zeros((n, z.is_("rho1_n_out")))
        for k in range(3):
            K = f"A{k + 1}"
            C = z.is_(K + "_n_rad_max")
            Rb = np.stack([self._radial(k, mu[bi[b]], mu[bj[b]], r[b] / rc[b]) for b in range(len(bi))]) if len(bi) else np.zeros((0, self.nl, C))
            msg_new = [None] * n
            if k > 0:
                nlmi = z.is_(K + "_n_lm_ind")
                cgw = z.f(K + "_cg_W").reshape(self.nlm * nlmi, -1)
                zproj = (self.chem @ z.f(K + "_chem_linear_W").reshape(self.emb, C)) * z.fs(K + "_chem_linear_norm", 1.0)
                mask = z.f(K + "_chem_l0_mask").reshape(-1)
            for i in range(n):
                sel = np.nonzero(bi == i)[0]
                U = Y[sel][:, :, None] * Rb[sel][:, l_of, :]                      # [bonds][lm][C]
                T = {}
                if k == 0:
                    T[K] = U.sum(0)
                    X = K
                else:
                    Ic = np.stack([msg_prev[j] for j in bj[sel]]) + mask[None, :, None] * zproj[mu[bj[sel]]][:, None, :] \
                        if len(sel) else np.zeros((0, nlmi, C))
                    P = np.einsum("byc,bic->yic", U, Ic).reshape(self.nlm * nlmi, C)
                    T[K] = cgw.T @ P
                    T[K + "_red"] = self._reduce(K + "_red", T, mu[i])
                    X = K + "_red"
                msg_new[i], rho = self._chain(k, T, X, mu[i])
                rho_sum[i] += rho
            msg_prev = msg_new
        W0, W1 = z.f("energy_mlp_W0"), z.f("energy_mlp_W1").reshape(-1)
        s = (rho_sum[:, 1:] @ W0) * z.fs("energy_mlp_norm0", 1.0)
        act = np.tanh(s) if z.is_("energy_mlp_activation", 0) == 1 else s / (1.0 + np.exp(-s))
        e = (act @ W1) * z.fs("energy_mlp_norm1", 1.0)
        energies = (e + rho_sum[:, 0]) * self.oscale + self.shift[mu]
        return dict(energy=float(energies.sum()), energies=energies)
