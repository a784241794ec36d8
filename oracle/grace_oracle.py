"""TEST INFRASTRUCTURE ONLY - numpy fp64 restatement of the reference's GRACE-1L / GRACE-2L evaluation path.

Nothing of the product imports this file: only tests/, the smoke check and the CPU-baseline leg of the benchmark
use it, as the checker.  Every function cites the reference file:line whose arithmetic it restates.

Differences from the reference CPU drivers, all below the parity tolerances:
  * everything is fp64 (the reference network is fp32 with fp64 geometry and sums);
  * the radial MLP is evaluated exactly per bond by default; ``spline_n > 0`` selects the reference's cubic Hermite
    tables (libgrace/src/fused_1l.cpp:102-129, libgrace/include/grace/fused_cpu.h:1052-1073);
  * the neighbour list is a brute-force image scan (same bond set as python/src/neighbors.cpp:15-95).
Pinned against the reference's own golden vectors (TensorFlow fp64, tests/fixtures/ref_tf/order3_tf.npz) and
against the compiled reference drivers in tests/test_oracle.py.
"""
from __future__ import annotations

import io
import zipfile

import numpy as np


# ----------------------------------------------------------------------------------------------------------------
# kokkos.npz access (libgrace/src/npz3.h:105-149: every array is read by its stored dtype)
# ----------------------------------------------------------------------------------------------------------------
class Npz:
    def __init__(self, path):
        self.a = {}
        with zipfile.ZipFile(path) as z:
            for name in z.namelist():
                key = name[:-4] if name.endswith(".npy") else name
                self.a[key] = np.load(io.BytesIO(z.read(name)), allow_pickle=False)

    def has(self, k):
        return k in self.a

    def f(self, k, default=None):
        if k not in self.a:
            if default is None:
                raise KeyError(k)
            return default
        return np.asarray(self.a[k], dtype=np.float64)

    def i(self, k, default=None):
        if k not in self.a:
            if default is None:
                raise KeyError(k)
            return default
        return np.asarray(self.a[k]).astype(np.int64)

    def fs(self, k, default=None):
        v = self.f(k, None if default is None else np.array([default]))
        return float(np.asarray(v).reshape(-1)[0])

    def is_(self, k, default=None):
        v = self.i(k, None if default is None else np.array([default]))
        return int(np.asarray(v).reshape(-1)[0])

    def names(self, k):
        if k not in self.a:
            return []
        return [x.decode() if isinstance(x, bytes) else str(x) for x in np.asarray(self.a[k]).reshape(-1)]


# ----------------------------------------------------------------------------------------------------------------
# radial part
# ----------------------------------------------------------------------------------------------------------------
def radial_basis(x, p, nrb):
    """g_k = T_k(2x-1) fc_p(x), k = 1..nrb, and d/dx (libgrace/include/grace/radial_x.h:11-26)."""
    x = np.asarray(x, dtype=np.float64)
    xp = x ** p
    xp1 = xp * x
    xp2 = xp1 * x
    fc = 1.0 - 0.5 * (p + 1) * (p + 2) * xp + p * (p + 2) * xp1 - 0.5 * p * (p + 1) * xp2
    dfc = 0.5 * p * (p + 1) * (p + 2) * (-(x ** (p - 1)) + 2.0 * xp - xp1)
    t = 2.0 * x - 1.0
    Tp, Tc, dTp, dTc = np.ones_like(x), t, np.zeros_like(x), 2.0 * np.ones_like(x)
    g = np.empty(x.shape + (nrb,))
    dg = np.empty_like(g)
    for k in range(nrb):
        g[..., k] = Tc * fc
        dg[..., k] = dTc * fc + Tc * dfc
        Tn = 2.0 * t * Tc - Tp
        dTn = 2.0 * (2.0 * Tc + t * dTc) - dTp
        Tp, dTp, Tc, dTc = Tc, dTc, Tn, dTn
    return g, dg


def mlp_forward_mode(layers, h, dh, act):
    """Radial MLP value and d/dx: hidden s = norm W^T h, SiLU (tanh if act == 1), no bias, linear output
    (libgrace/include/grace/radial_x.h:30-60).  layers: list of (W [n_in, n_out], norm)."""
    n = len(layers)
    for il, (W, norm) in enumerate(layers):
        s = (h @ W) * norm
        ds = (dh @ W) * norm
        if il < n - 1:
            if act == 1:
                s = np.tanh(s)
                ds = ds * (1.0 - s * s)
            else:
                sg = 1.0 / (1.0 + np.exp(-s))
                ds = sg * (1.0 + s * (1.0 - sg)) * ds
                s = s * sg
        h, dh = s, ds
    return h, dh


def radial_tables(layers, p, nrb, act, N):
    """Cubic Hermite coefficients [N, 4, nout] cast to fp32 as the reference stores them
    (libgrace/src/fused_1l.cpp:102-129)."""
    xk = np.arange(N + 1) / N
    g, dg = radial_basis(xk, p, nrb)
    f, d = mlp_forward_mode(layers, g, dg, act)
    d = d / N
    f0, f1, d0, d1 = f[:-1], f[1:], d[:-1], d[1:]
    c = np.stack([f0, d0, -3.0 * f0 - 2.0 * d0 + 3.0 * f1 - d1, 2.0 * f0 + d0 - 2.0 * f1 + d1], axis=1)
    return c.astype(np.float32).astype(np.float64)


def spline_eval(tab, x):
    """Value and d/dx by Horner on the table (libgrace/include/grace/fused_cpu.h:1052-1073)."""
    N = tab.shape[0]
    s = x * N
    k = np.clip(s.astype(np.int64), 0, N - 1)
    t = (s - k)[:, None]
    c = tab[k]
    R = c[:, 0] + t * (c[:, 1] + t * (c[:, 2] + t * c[:, 3]))
    dR = (c[:, 1] + t * (2.0 * c[:, 2] + t * 3.0 * c[:, 3])) * N
    return R, dR


# ----------------------------------------------------------------------------------------------------------------
# real spherical harmonics with gradient of the polynomial extension
# ----------------------------------------------------------------------------------------------------------------
def sph_harm(u, lmax):
    """Y [nb, nlm] and G = dY/d(x,y,z) [nb, nlm, 3]; Y00 = 1, lm = l(l+1)+m
    (libgrace/include/grace/fused_cpu.h:686-798)."""
    u = np.asarray(u, dtype=np.float64)
    nb = u.shape[0]
    rx, ry, rz = u[:, 0], u[:, 1], u[:, 2]
    nlm = (lmax + 1) ** 2
    npl = (lmax + 1) * (lmax + 2) // 2
    plm = np.zeros((npl, nb))
    dplm = np.zeros((npl, nb))
    plm[0] = 1.0
    if lmax > 0:
        plm[1] = np.sqrt(3.0) * rz
        dplm[1] = np.sqrt(3.0)
        plm[2] = -np.sqrt(1.5)
        for l in range(2, lmax + 1):
            for m in range(l - 1):
                idx, i1, i2 = l * (l + 1) // 2 + m, (l - 1) * l // 2 + m, (l - 2) * (l - 1) // 2 + m
                ca = np.sqrt((4.0 * l * l - 1.0) / (l * l - m * m))
                cb = -np.sqrt(((l - 1.0) ** 2 - m * m) / (4.0 * (l - 1.0) ** 2 - 1.0))
                plm[idx] = ca * (rz * plm[i1] + cb * plm[i2])
                dplm[idx] = ca * (plm[i1] + rz * dplm[i1] + cb * dplm[i2])
            prev, i0, i1 = (l - 1) * l // 2 + l - 1, l * (l + 1) // 2 + l - 1, l * (l + 1) // 2 + l
            sd, sc = np.sqrt(2.0 * l + 1.0), -np.sqrt(1.0 + 0.5 / l)
            plm[i0] = sd * plm[prev] * rz
            plm[i1] = sc * plm[prev]
            dplm[i0] = sd * (dplm[prev] * rz + plm[prev])
            dplm[i1] = sc * dplm[prev]
    Y = np.zeros((nb, nlm))
    G = np.zeros((nb, nlm, 3))
    sq2 = np.sqrt(2.0)
    for l in range(lmax + 1):
        c, p0 = l * (l + 1), l * (l + 1) // 2
        Y[:, c] = plm[p0]
        G[:, c, 2] = dplm[p0]
        pr, pi = rx.copy(), ry.copy()
        prx, pry, pix, piy = np.ones(nb), np.zeros(nb), np.zeros(nb), np.ones(nb)
        for m in range(1, l + 1):
            sg = sq2 if m % 2 == 0 else -sq2
            pv, dpv = plm[p0 + m], dplm[p0 + m]
            Y[:, c + m] = sg * pr * pv
            Y[:, c - m] = sg * pi * pv
            G[:, c + m, 0] = sg * prx * pv
            G[:, c + m, 1] = sg * pry * pv
            G[:, c + m, 2] = sg * pr * dpv
            G[:, c - m, 0] = sg * pix * pv
            G[:, c - m, 1] = sg * piy * pv
            G[:, c - m, 2] = sg * pi * dpv
            nrx = prx * rx + pr - pix * ry
            nry = pry * rx - piy * ry - pi
            nix = prx * ry + pix * rx + pi
            niy = pry * ry + pr + piy * rx
            prx, pry, pix, piy = nrx, nry, nix, niy
            pr, pi = pr * rx - pi * ry, pr * ry + pi * rx
    return Y, G


# ----------------------------------------------------------------------------------------------------------------
# neighbour list
# ----------------------------------------------------------------------------------------------------------------
def neighbor_list(pos, cell, pbc, rc):
    """All bonds i <- j with 0 <= |x_j - x_i + S cell| < rc, self-images included: arrays i, j, S [nb, 3]
    (bond set of python/src/neighbors.cpp:15-95; brute force over images)."""
    pos = np.asarray(pos, dtype=np.float64)
    cell = np.asarray(cell, dtype=np.float64).reshape(3, 3)
    n = len(pos)
    inv = np.linalg.inv(cell)
    h = 1.0 / np.linalg.norm(inv, axis=0)      # heights of the cell
    frac = pos @ inv
    reach = []
    for k in range(3):
        if pbc[k]:
            span = frac[:, k].max() - frac[:, k].min() if n else 0.0
            reach.append(int(np.ceil(rc / h[k] + span)) + 1)
        else:
            reach.append(0)
    ii, jj, SS = [], [], []
    rc2 = rc * rc
    for s0 in range(-reach[0], reach[0] + 1):
        for s1 in range(-reach[1], reach[1] + 1):
            for s2 in range(-reach[2], reach[2] + 1):
                sh = s0 * cell[0] + s1 * cell[1] + s2 * cell[2]
                d = pos[None, :, :] + sh - pos[:, None, :]
                r2 = (d * d).sum(-1)
                m = r2 < rc2
                if s0 == 0 and s1 == 0 and s2 == 0:
                    m &= ~np.eye(n, dtype=bool)
                a, b = np.nonzero(m)
                ii.append(a)
                jj.append(b)
                SS.append(np.tile(np.array([s0, s1, s2]), (len(a), 1)))
    i = np.concatenate(ii) if ii else np.zeros(0, dtype=np.int64)
    j = np.concatenate(jj) if jj else np.zeros(0, dtype=np.int64)
    S = np.concatenate(SS) if SS else np.zeros((0, 3), dtype=np.int64)
    order = np.lexsort((S[:, 2], S[:, 1], S[:, 0], j, i))
    return i[order], j[order], S[order]


# ----------------------------------------------------------------------------------------------------------------
# dense operators on [atom, function, channel] tensors
# ----------------------------------------------------------------------------------------------------------------
class FC:
    """out[f] = nof[f] (norm_l W_l[:, :, tile_l f]^T-contract Xl[f] + sum_{c -> f} norm_r W_r[:, :, tile_r c] Xr[from c])
    (libgrace/include/grace/fused_cpu.h:1103-1175, 349-364)."""

    def __init__(self, z, p):
        self.wl = z.f(p + "_w_left") * z.fs(p + "_norm_left", 1.0)       # [n_out, n_in_l, tiles]
        self.wr = z.f(p + "_w_right") * z.fs(p + "_norm_right", 1.0)
        self.tl = z.i(p + "_w_tile_left")
        self.tr = z.i(p + "_w_tile_right")
        self.to = z.i(p + "_collect_to")
        self.fr = z.i(p + "_collect_from")
        self.nof = z.f(p + "_norm_out_factor").reshape(-1)
        self.nf = len(self.tl)

    def fwd(self, Xl, Xr):
        out = np.einsum("afn,knf->afk", Xl[:, : self.nf], self.wl[:, :, self.tl])
        r = np.einsum("acn,knc->ack", Xr[:, self.fr], self.wr[:, :, self.tr])
        np.add.at(out, (slice(None), self.to), r)
        return out * self.nof[None, :, None]

    def bwd(self, g, nfl, nfr):
        g = g * self.nof[None, :, None]
        gl = np.zeros((g.shape[0], nfl, self.wl.shape[1]))
        gl[:, : self.nf] = np.einsum("afk,knf->afn", g, self.wl[:, :, self.tl])
        gr = np.zeros((g.shape[0], nfr, self.wr.shape[1]))
        np.add.at(gr, (slice(None), self.fr), np.einsum("ack,knc->acn", g[:, self.to], self.wr[:, :, self.tr]))
        return gl, gr


class Prod:
    """out[o] = sum_{t: msum_t = o} cg_t L[l_t] R[r_t], channel-wise (libgrace/include/grace/fused_cpu.h:1177-1198,
    411-453)."""

    def __init__(self, z, p):
        self.l = z.i(p + "_left_ind")
        self.r = z.i(p + "_right_ind")
        self.o = z.i(p + "_m_sum_ind")
        self.c = z.f(p + "_cg_coeff")
        self.nout = int(self.o.max()) + 1 if len(self.o) else 0

    def fwd(self, L, R):
        out = np.zeros((L.shape[0], self.nout, L.shape[2]))
        np.add.at(out, (slice(None), self.o), self.c[None, :, None] * L[:, self.l] * R[:, self.r])
        return out

    def bwd(self, L, R, g):
        gt = self.c[None, :, None] * g[:, self.o]
        gL = np.zeros_like(L)
        gR = np.zeros_like(R)
        np.add.at(gL, (slice(None), self.l), gt * R[:, self.r])
        np.add.at(gR, (slice(None), self.r), gt * L[:, self.l])
        return gL, gR


class Reduce:
    """out[fo] = sum_s norm_s sum_c W_s[mu, :, :, tile_c] X_s[ci_c]; scalar reduces send every connection to function 0
    (libgrace/include/grace/fused_cpu.h:1200-1273, 637-649)."""

    def __init__(self, z, prefix, sources, n_out, nfo, elem, scalar):
        self.src = []
        self.n_out, self.nfo, self.elem = n_out, nfo, elem
        for s in sources:
            if not z.has(f"{prefix}_reduce_{s}_W"):
                self.src.append(None)
                continue
            W = z.f(f"{prefix}_reduce_{s}_W") * z.fs(f"{prefix}_reduce_{s}_norm", 1.0)
            ci = z.i(f"{prefix}_collect_ind_{s}")
            tile = z.i(f"{prefix}_w_l_tile_{s}")
            if scalar or not z.has(f"{prefix}_total_sum_ind_{s}"):
                fo = np.zeros(len(ci), dtype=np.int64)
            else:
                fo = z.i(f"{prefix}_total_sum_ind_{s}").reshape(-1)
            if not elem:
                W = W[None]
            self.src.append((W, ci, tile, fo))

    def fwd(self, X, mu):
        na = X[0].shape[0]
        out = np.zeros((na, self.nfo, self.n_out))
        sel = mu if self.elem else np.zeros(na, dtype=np.int64)
        for S, x in zip(self.src, X):
            if S is None or x is None:
                continue
            W, ci, tile, fo = S
            for m in np.unique(sel):
                a = np.nonzero(sel == m)[0]
                r = np.einsum("acn,knc->ack", x[a][:, ci], W[m][:, :, tile])
                tmp = np.zeros((len(a), self.nfo, self.n_out))
                np.add.at(tmp, (slice(None), fo), r)
                out[a] += tmp
        return out

    def bwd(self, g, mu, shapes):
        na = g.shape[0]
        sel = mu if self.elem else np.zeros(na, dtype=np.int64)
        gX = []
        for S, shp in zip(self.src, shapes):
            if S is None or shp is None:
                gX.append(None)
                continue
            W, ci, tile, fo = S
            gx = np.zeros((na,) + shp)
            for m in np.unique(sel):
                a = np.nonzero(sel == m)[0]
                r = np.einsum("ack,knc->acn", g[a][:, fo], W[m][:, :, tile])
                tmp = np.zeros((len(a),) + shp)
                np.add.at(tmp, (slice(None), ci), r)
                gx[a] = tmp
            gX.append(gx)
        return gX


def _mlp_layers(z, prefix, n_layers):
    return [(z.f(f"{prefix}_W{i}"), z.fs(f"{prefix}_norm{i}", 1.0)) for i in range(n_layers)]


def _energy_mlp(z):
    n = z.is_("energy_mlp_n_layers", 2)
    layers = [[z.f(f"energy_mlp_W{i}").copy(), z.fs(f"energy_mlp_norm{i}", 1.0)] for i in range(n)]
    ln = z.has("energy_mlp_scale")
    if ln:      # legacy: RMS layer norm scale folded into layer 0 (libgrace/src/npz3.h:330-338)
        layers[0][0] = layers[0][0] * z.f("energy_mlp_scale").reshape(-1)[:, None]
    return layers, ln


def _energy_mlp_eval(layers, act, ln, x):
    """MLP value and gradient wrt its input x [na, nin] (libgrace/src/fused_1l.cpp:378-427,
    libgrace/include/grace/fused_cpu.h:664-681)."""
    na, nin = x.shape
    q = None
    x0 = x
    if ln:
        q = 1.0 / np.sqrt((x * x).mean(axis=1) + 1e-16)
        x = x * q[:, None]
    pre, h = [], x
    n = len(layers)
    for L, (W, norm) in enumerate(layers):
        v = (h @ W) * norm
        pre.append(v)
        if L < n - 1:
            h = np.tanh(v) if act == 1 else v / (1.0 + np.exp(-v))
        else:
            h = v
    val = h[:, 0]
    g = np.ones((na, 1))
    for L in range(n - 1, -1, -1):
        W, norm = layers[L]
        if L < n - 1:
            v = pre[L]
            if act == 1:
                t = np.tanh(v)
                g = g * (1.0 - t * t)
            else:
                sg = 1.0 / (1.0 + np.exp(-v))
                g = g * sg * (1.0 + v * (1.0 - sg))
        g = (g @ W.T) * norm
    if ln:
        t = (g * x0).sum(axis=1)
        g = q[:, None] * (g - x0 * (t * q * q / nin)[:, None])
    return val, g


def _l_of_lm(nlm):
    return np.floor(np.sqrt(np.arange(nlm) + 1e-9)).astype(np.int64)


class GraceOracle:
    """GRACE-1L / 2L energy, forces and virial of one structure (libgrace/src/fused_1l.cpp:260-427, 474-582;
    libgrace/src/fused_2l.cpp:410-781, 849-1099)."""

    def __init__(self, path, spline_n=0):
        z = self.z = Npz(path)
        kind = z.names("grace_model_kind")
        if kind:
            self.layers = {"GRACE-1L": 1, "GRACE-2L": 2}.get(kind[0], 0)
        else:
            self.layers = 2 if z.has("B0_lin_transform_W") else 1
        if self.layers == 0:
            raise ValueError("oracle: GRACE-1L / GRACE-2L only")
        self.spline_n = spline_n
        self.element_names = z.names("element_names")
        self.n_elements = z.is_("n_elements", 89)
        self.E = z.is_("embedding_size", 128)
        self.lmax = z.is_("lmax", 4)
        self.nl = self.lmax + 1
        self.nlm = self.nl ** 2
        self.nrb = z.is_("nradbase", 10)
        self.p = z.is_("radial_basis_p", 16)
        self.rcut = z.fs("rcut", 6.0)
        self.bond_rc = None
        if z.is_("has_bond_specific_cutoff", 0) and z.has("bond_cutoff_map"):
            self.bond_rc = z.f("bond_cutoff_map").reshape(self.n_elements, self.n_elements)
        self.chem = z.f("chem_embedding")
        self.rad_act = z.is_("radial_activation", 0)
        self.e_act = z.is_("energy_mlp_activation", 0 if self.layers == 1 else 1)
        self.e_layers, self.e_ln = _energy_mlp(z)
        self.scale = z.fs("output_scale", 1.0)
        self.shift = z.f("shift_values", np.zeros(self.n_elements)).reshape(-1)
        self.l_of = _l_of_lm(self.nlm)
        o4 = z.has("prod_AAAA_n_cg_terms")
        pre = "mlp_rad" if self.layers == 1 else "mlp_rad_R"
        self.rad1 = _mlp_layers(z, pre, z.is_(pre + "_n_layers", 3))
        self.zA = (self.chem @ z.f("A_lin_transform_W")) * z.fs("A_lin_transform_norm", 1.0) * \
            z.fs("A_inv_avg_n_neigh", 1.0)
        self.fcA1, self.pAA, self.fcAA1, self.pAAA = FC(z, "fc_A1"), Prod(z, "prod_AA"), FC(z, "fc_AA1"), \
            Prod(z, "prod_AAA")
        self.fcAA2 = FC(z, "fc_AA2") if o4 else None
        self.pAAAA = Prod(z, "prod_AAAA") if o4 else None
        self.aaa_a = bool(z.is_("AAA_right_A", 0)) if self.layers == 1 else True
        self.nrho = z.is_("rho_n_out", 17)
        src4 = ["A", "AA", "AAA", "AAAA"]
        self.rRho = Reduce(z, "rho", src4, self.nrho, 1, True, True)
        self.tab1 = self.tab2 = None
        if spline_n > 0:
            self.tab1 = radial_tables(self.rad1, self.p, self.nrb, self.rad_act, spline_n)
        if self.layers == 2:
            self.rad2 = _mlp_layers(z, "mlp_rad_R1", z.is_("mlp_rad_R1_n_layers", 3))
            if spline_n > 0:
                self.tab2 = radial_tables(self.rad2, self.p, self.nrb, self.rad_act, spline_n)
            self.zB0 = (self.chem @ z.f("B0_lin_transform_W")) * z.fs("B0_lin_transform_norm", 1.0) * \
                z.fs("B0_inv_avg_n_neigh", 1.0)
            self.nI1, self.nI = z.is_("I1_n_funcs", 4), z.is_("I_n_funcs", 4)
            self.rI1 = Reduce(z, "I1", src4, z.is_("I1_n_out", 12), self.nI1, True, False)
            self.rI = Reduce(z, "I", ["I1"], z.is_("I_n_out", 32), self.nI, False, False)
            self.CR = z.is_("I_n_out", 32)
            lr = z.i("YI_lr_inds").reshape(-1, 2)
            self.yi_y, self.yi_i = lr[:, 0], lr[:, 1]
            self.yi_o = z.i("YI_m_sum_ind")
            self.yi_c = z.f("YI_cg_coeff") * z.fs("YI_inv_avg_n_neigh", 1.0)
            self.nYI = int(self.yi_o.max()) + 1
            self.nB = z.is_("B_n_funcs", 31)
            self.rB = Reduce(z, "B", ["YI", "B0"], z.is_("B_n_out", 64), self.nB, False, False)
            o4b = z.has("prod_BBBB_n_cg_terms")
            self.fcB1, self.pBB, self.fcBB1, self.pBBB = FC(z, "fc_B1"), Prod(z, "prod_BB"), FC(z, "fc_BB1"), \
                Prod(z, "prod_BBB")
            self.fcBB2 = FC(z, "fc_BB2") if o4b else None
            self.pBBBB = Prod(z, "prod_BBBB") if o4b else None
            self.nI2 = z.is_("I2_n_out", 17)
            self.rI2 = Reduce(z, "I2", ["B", "BB", "BBB", "BBBB"], self.nI2, 1, True, True)
            self.rms = bool(z.is_("energy_rms_norm", 1))
            if self.rms:
                self.lnI = z.f("I_nl_LN_scale").reshape(-1)
                self.ln0 = z.f("I_0_LN_scale").reshape(-1)
            else:
                self.lnI = np.ones(self.nrho - 1)
                self.ln0 = np.ones(self.nI2)

        # UQ head of schema 6 (libgrace/src/uq_head.cpp:12-78), optional
        self.uq = None
        if z.is_("uq_schema_version", 0) == 6:
            E, K, D = self.n_elements, z.is_("uq_max_clusters"), z.is_("uq_feature_dim")
            self.uq = dict(RP=z.is_("uq_rp_dim"), D=D, K=K, scale=z.fs("uq_rp_density_scale", 1.0),
                           R=z.f("uq_rp_matrix"), cen=z.f("uq_centroids").reshape(E, K, D),
                           icov=z.f("uq_inv_cov").reshape(E, K, D, D), ncl=z.i("uq_n_clusters").reshape(-1),
                           thr=z.f("uq_interp_thresholds").reshape(E, K))

    @staticmethod
    def _uq_basis(red, X):
        """Collected inputs of a scalar reduce per atom, each source flattened channel-major over its collected
        functions (libgrace/include/grace/fused_cpu.h:1291-1305; libgrace/include/grace/uq.h:1-9)."""
        cols = []
        for S, x in zip(red.src, X):
            if S is None or x is None:
                continue
            ci = S[1]
            cols.append(np.transpose(x[:, ci, :], (0, 2, 1)).reshape(len(x), -1))
        return np.concatenate(cols, axis=1)

    def _uq_eval(self, blocks, mu):
        """blocks: per-atom bases in the order of the projection matrix's rows, last layer first.  Returns gamma, sigma,
        cluster (libgrace/include/grace/fused_cpu.h:1378-1412; libgrace/src/fused_2l.cpp:1172-1184)."""
        u = self.uq
        B = np.concatenate(blocks, axis=1)
        n2 = [(b * b).sum(1) for b in blocks]
        nrm = np.sqrt(sum(n2))
        dens = [nrm, np.sqrt(n2[0])] + ([np.sqrt(n2[1])] if len(blocks) == 2 else [])
        f = np.concatenate([(B @ u["R"]) / (nrm + 1e-12)[:, None]] +
                           [(np.log(d + 1e-12) * u["scale"])[:, None] for d in dens], axis=1)
        n = len(mu)
        gamma, sigma, cluster = np.zeros(n), np.zeros(n), np.zeros(n)
        for a in range(n):
            m = mu[a]
            d = f[a][None, :] - u["cen"][m, :u["ncl"][m]]
            k = int(np.argmin((d * d).sum(1)))
            sig = np.sqrt(d[k] @ u["icov"][m, k] @ d[k] + 1e-8)
            sigma[a], gamma[a], cluster[a] = sig, sig / max(u["thr"][m, k], 1e-10), k
        return gamma, sigma, cluster

    # -- helpers -------------------------------------------------------------------------------------------------
    def cutoff_matrix(self, mus):
        if self.bond_rc is None:
            return np.full((len(mus), len(mus)), self.rcut)
        return self.bond_rc[np.ix_(mus, mus)]

    def _radial(self, layers, tab, x):
        if tab is not None:
            return spline_eval(tab, x)
        g, dg = radial_basis(x, self.p, self.nrb)
        return mlp_forward_mode(layers, g, dg, self.rad_act)

    @staticmethod
    def _scatter(Y, Rz, i, n, l_of):
        """X[i, lm, c] = sum_bonds Y[lm] (R[c, l(lm)] z[c]) (libgrace/include/grace/fused_cpu.h:947-982)."""
        X = np.zeros((n, Y.shape[1], Rz.shape[1]))
        np.add.at(X, i, Y[:, :, None] * Rz[:, :, l_of].transpose(0, 2, 1))
        return X

    def _chain_fwd(self, X0, fc1, pXX, fcXX1, pXXX, fcXX2, pXXXX, right_is_x0):
        X1 = fc1.fwd(X0, X0)
        XX = pXX.fwd(X1, X1)
        XX1 = fcXX1.fwd(XX, X0)
        Rr = X0 if right_is_x0 else X1
        XXX = pXXX.fwd(XX1, Rr)
        XX2 = fcXX2.fwd(XX, X0) if fcXX2 is not None else None
        XXXX = pXXXX.fwd(XX2, XX2) if pXXXX is not None else None
        return dict(X0=X0, X1=X1, XX=XX, XX1=XX1, XXX=XXX, XX2=XX2, XXXX=XXXX)

    def _chain_bwd(self, T, g, fc1, pXX, fcXX1, pXXX, fcXX2, pXXXX, right_is_x0):
        """g: gradients wrt (X0, XX, XXX, XXXX) from the reduces -> gradient wrt X0
        (libgrace/src/fused_1l.cpp:306-349)."""
        gX0, gXX, gXXX, gXXXX = g
        X0, X1, XX, XX1, XX2 = T["X0"], T["X1"], T["XX"], T["XX1"], T["XX2"]
        nf0, nfXX = X0.shape[1], XX.shape[1]
        gX1 = np.zeros_like(X1)
        if pXXXX is not None and gXXXX is not None:
            gl, gr = pXXXX.bwd(XX2, XX2, gXXXX)
            a, b = fcXX2.bwd(gl + gr, nfXX, nf0)
            gXX = gXX + a
            gX0 = gX0 + b
        Rr = X0 if right_is_x0 else X1
        gl, gr = pXXX.bwd(XX1, Rr, gXXX)
        if right_is_x0:
            gX0 = gX0 + gr
        else:
            gX1 = gX1 + gr
        a, b = fcXX1.bwd(gl, nfXX, nf0)
        gXX = gXX + a
        gX0 = gX0 + b
        gl, gr = pXX.bwd(X1, X1, gXX)
        gX1 = gX1 + gl + gr
        a, b = fc1.bwd(gX1, nf0, nf0)
        return gX0 + a + b

    # -- the evaluation ----------------------------------------------------------------------------------------
    def compute(self, species, types, pos, cell, pbc, bonds=None, uq=False):
        """species: element names of types 1..len(species); returns dict(energy, forces, virial, energies) and, with
        uq, gamma / sigma / cluster per atom."""
        if uq and self.uq is None:
            raise ValueError("the model has no UQ head")
        pos = np.asarray(pos, dtype=np.float64)
        cell = np.asarray(cell, dtype=np.float64).reshape(3, 3)
        n = len(pos)
        t2m = np.array([self.element_names.index(s) for s in species], dtype=np.int64)
        mu = t2m[np.asarray(types, dtype=np.int64) - 1]
        rcm = self.cutoff_matrix(np.arange(self.n_elements))
        if bonds is None:
            bonds = neighbor_list(pos, cell, pbc, rcm[np.ix_(t2m, t2m)].max())
        bi, bj, S = bonds
        d = pos[bj] - pos[bi] + S @ cell
        r = np.sqrt((d * d).sum(-1))
        rc = rcm[mu[bi], mu[bj]]
        keep = r < rc
        if np.any(r[keep] == 0.0):
            raise ValueError("two atoms at the same position")
        bi, bj, d, r, rc = bi[keep], bj[keep], d[keep], r[keep], rc[keep]
        u = d / r[:, None]
        x = r / rc
        Y, G = sph_harm(u, self.lmax)
        nl, l_of = self.nl, self.l_of
        # layer 1
        R, dR = self._radial(self.rad1, self.tab1, x)
        C1 = self.zA.shape[1]
        R = R.reshape(-1, C1, nl)
        dR = dR.reshape(-1, C1, nl)
        zj = self.zA[mu[bj]]
        A = self._scatter(Y, R * zj[:, :, None], bi, n, l_of)
        ra = self.aaa_a
        T1 = self._chain_fwd(A, self.fcA1, self.pAA, self.fcAA1, self.pAAA, self.fcAA2, self.pAAAA, ra)
        X1 = [T1["X0"], T1["XX"], T1["XXX"], T1["XXXX"]]
        rho = self.rRho.fwd(X1, mu)[:, 0]
        shapes1 = [None if t is None else t.shape[1:] for t in X1]
        fv = np.zeros((len(bi), 3))

        def bond_bwd(gX, Rl, dRl, zl, extra_gR=None, extra_gY=None):
            """per-bond dE/dx and dE/dY -> force on i (libgrace/include/grace/fused_cpu.h:836-860, 1027-1050)."""
            gXb = gX[bi]                                           # [nb, nlm, C]
            Rz = (Rl * zl[:, :, None])[:, :, l_of].transpose(0, 2, 1)    # [nb, nlm, C]
            gY = (gXb * Rz).sum(-1)
            gRlm = Y[:, :, None] * gXb * zl[:, None, :]            # [nb, nlm, C]
            gR = np.zeros((len(bi), Rl.shape[1], nl))
            for l in range(nl):
                gR[:, :, l] = gRlm[:, l * l:(l + 1) * (l + 1)].sum(1)
            if extra_gR is not None:
                gR = gR + extra_gR
            if extra_gY is not None:
                gY = gY + extra_gY
            dEdx = (gR * dRl).sum((1, 2))
            gv = np.einsum("bq,bqd->bd", gY, G)
            gr_ = (gv * u).sum(-1)
            return (dEdx / rc)[:, None] * u + (gv - gr_[:, None] * u) / r[:, None]

        if self.layers == 1:
            val, g = _energy_mlp_eval(self.e_layers, self.e_act, self.e_ln, rho[:, 1:])
            e_atom = (val + rho[:, 0]) * self.scale + self.shift[mu]
            grho = np.concatenate([np.full((n, 1), self.scale), g * self.scale], axis=1)
            gX = self.rRho.bwd(grho[:, None, :], mu, shapes1)
            gX = [np.zeros((n,) + s) if (g_ is None and s is not None) else g_ for g_, s in zip(gX, shapes1)]
            gA = self._chain_bwd(T1, gX, self.fcA1, self.pAA, self.fcAA1, self.pAAA, self.fcAA2, self.pAAAA, ra)
            fv += bond_bwd(gA, R, dR, zj)
        else:
            I1 = self.rI1.fwd(X1, mu)
            I = self.rI.fwd([I1], mu)                               # [n, nI, CR]
            CR = self.CR
            R1, dR1 = self._radial(self.rad2, self.tab2, x)
            R1 = R1.reshape(-1, CR, nl)
            dR1 = dR1.reshape(-1, CR, nl)
            zb = self.zB0[mu[bj]]
            B0 = self._scatter(Y, R1 * zb[:, :, None], bi, n, l_of)
            # YI[o] = inv_avg sum_t cg_t sum_j Y[y_t] R1[l(y_t)] I_j[i_t] (libgrace/src/fused_2l.cpp:229-276,646-651)
            ly = l_of[self.yi_y]
            Ij = I[bj]                                              # [nb, nI, CR]
            YI = np.zeros((n, self.nYI, CR))
            for t in range(len(self.yi_o)):
                contrib = self.yi_c[t] * Y[:, self.yi_y[t], None] * R1[:, :, ly[t]] * Ij[:, self.yi_i[t]]
                np.add.at(YI[:, self.yi_o[t]], bi, contrib)
            B = self.rB.fwd([YI, B0], mu)
            T2 = self._chain_fwd(B, self.fcB1, self.pBB, self.fcBB1, self.pBBB, self.fcBB2, self.pBBBB, True)
            X2 = [T2["X0"], T2["XX"], T2["XXX"], T2["XXXX"]]
            I2 = self.rI2.fwd(X2, mu)[:, 0]
            # readout (libgrace/src/fused_2l.cpp:548-615)
            nr = self.nrho
            eps = 1e-10
            s1 = np.sqrt((rho[:, 1:] ** 2).sum(1) / (nr - 1) + eps) if self.rms else np.ones(n)
            s0 = np.sqrt((I2 ** 2).sum(1) / self.nI2 + eps) if self.rms else np.ones(n)
            xin = rho[:, 1:] / s1[:, None] * self.lnI + I2[:, 1:] / s0[:, None] * self.ln0[1:]
            val, g = _energy_mlp_eval(self.e_layers, self.e_act, self.e_ln, xin)
            e_atom = (val + rho[:, 0] + I2[:, 0] / s0 * self.ln0[0]) * self.scale + self.shift[mu]
            g = g * self.scale
            grho = np.zeros((n, nr))
            grho[:, 0] = self.scale
            t1 = (g * self.lnI * rho[:, 1:]).sum(1) if self.rms else np.zeros(n)
            grho[:, 1:] = g * self.lnI / s1[:, None] - rho[:, 1:] * (t1 / ((nr - 1) * s1 ** 3))[:, None]
            gy = np.concatenate([np.full((n, 1), self.scale), g], axis=1)
            t0 = (gy * self.ln0 * I2).sum(1) if self.rms else np.zeros(n)
            gI2 = gy * self.ln0 / s0[:, None] - I2 * (t0 / (self.nI2 * s0 ** 3))[:, None]
            # layer-2 reverse
            shapes2 = [None if t is None else t.shape[1:] for t in X2]
            gX = self.rI2.bwd(gI2[:, None, :], mu, shapes2)
            gX = [np.zeros((n,) + s) if (g_ is None and s is not None) else g_ for g_, s in zip(gX, shapes2)]
            gB = self._chain_bwd(T2, gX, self.fcB1, self.pBB, self.fcBB1, self.pBBB, self.fcBB2, self.pBBBB, True)
            gYI, gB0 = self.rB.bwd(gB, mu, [YI.shape[1:], B0.shape[1:]])
            extra_gR = np.zeros((len(bi), CR, nl))
            extra_gY = np.zeros((len(bi), self.nlm))
            gI = np.zeros_like(I)
            for t in range(len(self.yi_o)):
                go = self.yi_c[t] * gYI[bi, self.yi_o[t]]            # [nb, CR]
                yv, rl, ij = Y[:, self.yi_y[t]], R1[:, :, ly[t]], Ij[:, self.yi_i[t]]
                extra_gY[:, self.yi_y[t]] += (go * rl * ij).sum(-1)
                extra_gR[:, :, ly[t]] += yv[:, None] * go * ij
                np.add.at(gI[:, self.yi_i[t]], bj, yv[:, None] * go * rl)
            fv += bond_bwd(gB0, R1, dR1, zb, extra_gR, extra_gY)
            # layer-1 reverse seeded with dE/dI and dE/drho (libgrace/src/fused_2l.cpp:459-542)
            (gI1,) = self.rI.bwd(gI, mu, [I1.shape[1:]])
            gXa = self.rI1.bwd(gI1, mu, shapes1)
            gXb = self.rRho.bwd(grho[:, None, :], mu, shapes1)
            gX = []
            for a_, b_, s in zip(gXa, gXb, shapes1):
                if s is None:
                    gX.append(None)
                else:
                    gX.append((a_ if a_ is not None else 0.0) + (b_ if b_ is not None else np.zeros((n,) + s)))
            gA = self._chain_bwd(T1, gX, self.fcA1, self.pAA, self.fcAA1, self.pAAA, self.fcAA2, self.pAAAA, True)
            fv += bond_bwd(gA, R, dR, zj)
        forces = np.zeros((n, 3))
        np.add.at(forces, bi, fv)
        np.add.at(forces, bj, -fv)
        # virial += (x_i - x_j) (x) fv, order xx yy zz xy xz yz (libgrace/src/fused_1l.cpp:45-51)
        dl = -d
        vir = np.array([(dl[:, 0] * fv[:, 0]).sum(), (dl[:, 1] * fv[:, 1]).sum(), (dl[:, 2] * fv[:, 2]).sum(),
                        (dl[:, 0] * fv[:, 1]).sum(), (dl[:, 0] * fv[:, 2]).sum(), (dl[:, 1] * fv[:, 2]).sum()])
        res = dict(energy=float(e_atom.sum()), forces=forces, virial=vir, energies=e_atom)
        if uq:
            blocks = [self._uq_basis(self.rRho, X1)]
            if self.layers == 2:
                blocks.insert(0, self._uq_basis(self.rI2, X2))
            res["gamma"], res["sigma"], res["cluster"] = self._uq_eval(blocks, mu)
        return res
