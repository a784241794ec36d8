"""GRACE-3L model files: the generator (grace_runtime_b200/modelgen3l.py) and the library's reader (csrc/model3l.cpp).

The reference tree ships no GRACE-3L model, so the generator builds the architecture tables itself (Gaunt couplings of the
real spherical harmonics the engines use).  What pins it: the reference's own loader and CPU engine accept the file and
the energy is invariant under rotations, with forces that match finite differences (compiled reference, when built).
The reader is checked on the same files and on malformed variants, where it has to name the array the reference's
loader names (libgrace/src/model_3l.cpp:36-154, 165-464).  GPU: energies, forces and virial of the library against the
compiled reference on generated models."""
import numpy as np
import pytest

from grace_runtime_b200 import modelgen3l


@pytest.fixture(scope="module")
def small3l(tmp_path_factory):
    return modelgen3l.write_model_3l(str(tmp_path_factory.mktemp("m3") / "small.npz"), elements=("Al", "Ni"), lmax=2,
                                     channels=(16, 16, 16))


def _cluster(n=12, seed=3):
    rng = np.random.default_rng(seed)
    pos = rng.uniform(-3.0, 3.0, (n, 3))
    types = rng.integers(1, 3, n).astype(np.int32)
    return types, pos


def test_real_sh_is_the_engines_convention():
    from oracle.grace_oracle import sph_harm
    rng = np.random.default_rng(0)
    u = rng.standard_normal((64, 3))
    u /= np.linalg.norm(u, axis=1)[:, None]
    assert np.abs(modelgen3l.real_sh(u, 4) - sph_harm(u, 4)[0]).max() < 1e-13


def test_gaunt_tensor():
    G = modelgen3l.gaunt(3)
    n = G.shape[0]
    assert np.allclose(G[0], np.eye(n), atol=1e-13)              # Y_00 = 1: orthonormality of the others
    assert np.allclose(G, G.transpose(1, 0, 2)) and np.allclose(G, G.transpose(2, 1, 0))
    l = modelgen3l._lm_l(3)
    odd = (l[:, None, None] + l[None, :, None] + l[None, None, :]) % 2 == 1
    assert np.all(G[odd] == 0.0)                                 # parity
    far = l[:, None, None] > l[None, :, None] + l[None, None, :]
    assert np.all(G[far] == 0.0)                                 # triangle rule


def test_reference_accepts_generated_model(small3l):
    from oracle import refcpu
    if not refcpu.available():
        pytest.skip("oracle/_ref is not built")
    m = refcpu.RefModel(small3l, ["Al", "Ni"])
    assert m.layers == 3 and abs(m.cutoff - 5.0) < 1e-12
    types, pos = _cluster()
    box, open_ = np.eye(3) * 60.0, [0, 0, 0]
    r = m.compute(types, pos + 30.0, box, open_)
    assert np.isfinite(r["energy"]) and np.abs(r["forces"]).max() > 1e-3
    assert np.abs(r["forces"].sum(0)).max() < 1e-5
    # rotation invariance (the couplings are Gaunt coefficients of the engine's harmonics)
    rng = np.random.default_rng(5)
    Q, _ = np.linalg.qr(rng.standard_normal((3, 3)))
    if np.linalg.det(Q) < 0:
        Q[:, 0] *= -1
    r2 = m.compute(types, pos @ Q.T + 30.0, box, open_)
    assert abs(r2["energy"] - r["energy"]) < 2e-5 * max(1.0, abs(r["energy"]))
    assert np.abs(r2["forces"] - r["forces"] @ Q.T).max() < 2e-4
    # forces against central differences of the energy (fp32 network: a wide step)
    h = 2e-3
    for i, d in ((0, 0), (5, 2)):
        p = pos + 30.0
        p[i, d] += h
        ep = m.compute(types, p, box, open_)["energy"]
        p[i, d] -= 2 * h
        em = m.compute(types, p, box, open_)["energy"]
        assert abs(-(ep - em) / (2 * h) - r["forces"][i, d]) < 5e-3 * max(1.0, np.abs(r["forces"]).max())


def test_reference_accepts_benchmark_shape(tmp_path):
    """lmax 4, 64 channels, 89 elements: the shape class of the 3L benchmark configuration."""
    from oracle import refcpu
    if not refcpu.available():
        pytest.skip("oracle/_ref is not built")
    from grace_runtime_b200 import modelgen, structures
    p = modelgen3l.write_model_3l(str(tmp_path / "big.npz"), elements=modelgen.ELEMENTS, lmax=4, channels=(64, 64, 64),
                                  rho_width=32, embedding=16, radial_hidden=128, energy_hidden=64, rcut=6.0, avg_neigh=58.0)
    species = modelgen._subset(2024, 5)
    types, pos, cell, pbc = structures.crystal("bcc", 3.2, (4, 4, 4), n_species=5, sigma=0.05, seed=1)
    r = refcpu.RefModel(p, species).compute(types, pos, cell, pbc)
    assert np.isfinite(r["energy"]) and np.abs(r["forces"].sum(0)).max() < 1e-4


def _load_error(path):
    from grace_runtime_b200 import backend as B
    with pytest.raises(ValueError) as e:
        B.Model(path)
    return str(e.value)


def test_library_reads_generated_model(small3l):
    from grace_runtime_b200 import backend as B
    m = B.Model(small3l)
    assert m.layers == 3 and m.element_names == ["Al", "Ni"] and not m.has_uq


def _variant(src, dst, edit):
    z = dict(np.load(src))
    edit(z)
    np.savez(dst, **z)
    return dst


def _drop(key):
    return lambda z: z.pop(key)


def _set(key, value):
    def f(z):
        z[key] = value
    return f


def _names(v):
    return np.array([s.encode() for s in v])


MALFORMED = [
    ("A2_cg_W", _drop("A2_cg_W")),
    ("A2_cg_W", lambda z: z.__setitem__("A2_cg_W", z["A2_cg_W"][:-1])),
    ("A2_chem_l0_mask", _set("A2_n_lm_ind", np.array([4]))),
    ("A1_nfunc", _set("A1_equivariant", np.array([1]))),
    ("A3_lin_transform_W", _set("A3_equivariant", np.array([0]))),
    ("A1_mlp_W1", lambda z: z.__setitem__("A1_mlp_W1", z["A1_mlp_W1"][:-1])),
    ("A1_mlp_b0", lambda z: z.__setitem__("A1_mlp_b0", z["A1_mlp_b0"][:-1])),
    ("A1_l_tile", lambda z: z.__setitem__("A1_l_tile", z["A1_l_tile"] + 1)),
    ("prod_names", lambda z: z.__setitem__("prod_names", z["prod_names"][:-1])),
    ("prod_names", lambda z: z.__setitem__("prod_names", np.concatenate([z["prod_names"], z["prod_names"][:1]]))),
    ("extra_n_out", lambda z: z.__setitem__("reduce_names", np.concatenate([z["reduce_names"], _names(["extra"])]))),
    ("A1_2_left_ind", lambda z: z.__setitem__("A1_2_left_ind", z["A1_2_left_ind"] + 100)),
    ("A1_2_m_sum_ind", lambda z: z.__setitem__("A1_2_m_sum_ind", z["A1_2_m_sum_ind"][:-1])),
    ("A1_3_U", _set("A1_3_n_left", np.array([8]))),
    ("A1_2_red_n_in_A1_3", _set("A1_2_red_instruction_names", _names(["A1_3"]))),
    ("A1_2_red_collect_ind_A1_2", lambda z: z.__setitem__("A1_2_red_collect_ind_A1_2", z["A1_2_red_collect_ind_A1_2"] + 1000)),
    ("fc_A2_2a_w_right", lambda z: z.__setitem__("fc_A2_2a_w_right", z["fc_A2_2a_w_right"][:, :-1])),
    ("fc_A1_2b_collect_to", lambda z: z.__setitem__("fc_A1_2b_collect_to", z["fc_A1_2b_collect_to"] + 9)),
    ("eq1_norm_l0_mask", lambda z: z.__setitem__("eq1_norm_degree_weights", z["eq1_norm_degree_weights"][:-1])),
    ("eq2_norm_expand_index", lambda z: z.__setitem__("eq2_norm_expand_index", z["eq2_norm_expand_index"] + 3)),
    ("rho2_norm_scale", lambda z: z.__setitem__("rho2_norm_scale", z["rho2_norm_scale"][:-1])),
    ("rho3_reduce_A3_red_W", lambda z: z.__setitem__("rho3_reduce_A3_red_W", z["rho3_reduce_A3_red_W"][:-1])),
    ("out1_origins", _set("out1_origins", _names(["rho1_norm", "rho2_norm"]))),
    ("energy_mlp_W0", lambda z: z.__setitem__("energy_mlp_W0", z["energy_mlp_W0"][:-1])),
    ("energy_rms_norm", _set("energy_rms_norm", np.array([1]))),
    ("shift_values", lambda z: z.__setitem__("shift_values", z["shift_values"][:-1])),
    # the layer graph
    ("spbf_names", _set("spbf_names", _names(["A1", "A3", "A2"]))),
    ("fc_names", lambda z: z.__setitem__("fc_names", z["fc_names"][:-1])),
    ("eq1_norm_affine_weight", lambda z: z.__setitem__("eq1_norm_affine_weight", z["eq1_norm_affine_weight"][:, :-1])),
    ("rho2_norm_n_out", lambda z: (z.__setitem__("rho2_norm_n_out", np.array([15])),
                                   z.__setitem__("rho2_norm_scale", z["rho2_norm_scale"][:-1]))),
    ("eqnorm_names", lambda z: z.__setitem__("eqnorm_names", z["eqnorm_names"][:1])),
]


@pytest.mark.parametrize("case", range(len(MALFORMED)))
def test_malformed_files_name_the_array(small3l, tmp_path, case):
    key, edit = MALFORMED[case]
    bad = _variant(small3l, str(tmp_path / "bad.npz"), edit)
    msg = _load_error(bad)
    assert key in msg, msg
    from oracle import refcpu
    if refcpu.available():      # the reference's loader rejects the same file, naming the same array
        with pytest.raises(RuntimeError) as e:
            refcpu.RefModel(bad, ["Al", "Ni"])
        assert key in str(e.value), str(e.value)


def test_numpy_restatement_matches_compiled_reference(small3l):
    """oracle/grace3l_oracle.py (forward pass, fp64) against the reference's CPU engine: periodic cell and open cluster."""
    from oracle import refcpu
    from oracle.grace3l_oracle import Grace3LOracle
    if not refcpu.available():
        pytest.skip("oracle/_ref is not built")
    rng = np.random.default_rng(1)
    a = 4.0
    base = np.array([[0, 0, 0], [.5, .5, 0], [.5, 0, .5], [0, .5, .5]]) * a
    pos = np.concatenate([base + np.array([i, j, 0]) * a for i in range(2) for j in range(2)])
    pos += 0.1 * rng.standard_normal(pos.shape)
    types = rng.integers(1, 3, len(pos)).astype(np.int32)
    ref, orc = refcpu.RefModel(small3l, ["Al", "Ni"]), Grace3LOracle(small3l)
    for cell, pbc, x in ((np.diag([2 * a, 2 * a, a]), [1, 1, 1], pos), (np.eye(3) * 50.0, [0, 0, 0], pos + 20.0)):
        r, o = ref.compute(types, x, cell, pbc), orc.compute(["Al", "Ni"], types, x, cell, pbc)
        assert np.abs(r["energies"] - o["energies"]).max() < 2e-6
        assert abs(r["energy"] - o["energy"]) / len(x) < 2e-7


def _cells():
    rng = np.random.default_rng(11)
    a = 4.0
    base = np.array([[0, 0, 0], [.5, .5, 0], [.5, 0, .5], [0, .5, .5]]) * a
    fcc = np.concatenate([base + np.array([i, j, k]) * a for i in range(2) for j in range(2) for k in range(2)])
    fcc += 0.12 * rng.standard_normal(fcc.shape)
    yield "fcc32", rng.integers(1, 3, len(fcc)).astype(np.int32), fcc, np.eye(3) * 2 * a, [1, 1, 1]
    tri = np.array([[5.1, 0.2, 0.0], [1.3, 4.7, 0.1], [0.4, 0.9, 5.3]])
    pos = rng.random((9, 3)) @ tri
    yield "tri9", rng.integers(1, 3, 9).astype(np.int32), pos, tri, [1, 1, 1]
    types, cl = _cluster(14, seed=8)
    yield "cluster14", types, cl + 30.0, np.eye(3) * 60.0, [0, 0, 0]
    yield "atom1", np.array([2], dtype=np.int32), np.array([[1.0, 2.0, 3.0]]), np.eye(3) * 40.0, [0, 0, 0]


@pytest.mark.gpu
def test_gpu_matches_compiled_reference(backend, small3l):
    """Energy, per-atom energies, forces and virial of the library against the reference's CPU engine."""
    from oracle import refcpu
    if not refcpu.available():
        pytest.skip("oracle/_ref is not built")
    ref = refcpu.RefModel(small3l, ["Al", "Ni"])
    sysm = backend.System(backend.Model(small3l), ["Al", "Ni"])
    for name, types, pos, cell, pbc in _cells():
        r = ref.compute(types, pos, cell, pbc)
        g = sysm.compute(types, pos, cell, pbc, energies=True)
        n = len(types)
        assert abs(g["energy"] - r["energy"]) / n < 2e-6, name
        assert np.abs(g["energies"] - r["energies"]).max() < 5e-6, name
        assert np.abs(g["forces"] - r["forces"]).max() < 2e-5 * max(1.0, np.abs(r["forces"]).max()), name
        assert np.abs(g["virial"] - r["virial"]).max() < 2e-5 * max(1.0, np.abs(r["virial"]).max()), name
        e_only = sysm.compute(types, pos, cell, pbc, energy_only=True)
        # (the couple of the bond sums adds in shared memory in no fixed order: fp32 rounding differs from run to run)
        assert abs(e_only["energy"] - g["energy"]) < 1e-7 * max(1.0, abs(g["energy"])), name


@pytest.mark.gpu
def test_gpu_forces_are_the_gradient(backend, small3l):
    sysm = backend.System(backend.Model(small3l), ["Al", "Ni"])
    name, types, pos, cell, pbc = next(_cells())
    g = sysm.compute(types, pos, cell, pbc)
    assert np.abs(g["forces"].sum(0)).max() < 1e-5
    h = 2e-3
    for i, d in ((0, 0), (7, 1), (20, 2)):
        p = pos.copy()
        p[i, d] += h
        ep = sysm.compute(types, p, cell, pbc, energy_only=True)["energy"]
        p[i, d] -= 2 * h
        em = sysm.compute(types, p, cell, pbc, energy_only=True)["energy"]
        assert abs(-(ep - em) / (2 * h) - g["forces"][i, d]) < 5e-3 * max(1.0, np.abs(g["forces"]).max())


@pytest.mark.gpu
def test_gpu_batch_and_larger_shape(backend, small3l, tmp_path):
    """A Batch of the cells, and a model with lmax 3 and 32 / 16 / 32 channels."""
    from oracle import refcpu
    if not refcpu.available():
        pytest.skip("oracle/_ref is not built")
    cells = list(_cells())
    ref = refcpu.RefModel(small3l, ["Al", "Ni"])
    batch = backend.Batch(backend.Model(small3l), ["Al", "Ni"])
    nat = np.array([len(c[1]) for c in cells], dtype=np.int32)
    res = batch.compute(nat, np.concatenate([c[1] for c in cells]), np.concatenate([c[2] for c in cells]),
                        np.stack([c[3] for c in cells]), np.array([c[4] for c in cells], dtype=np.uint8))
    at = 0
    for k, (name, types, pos, cell, pbc) in enumerate(cells):
        r = ref.compute(types, pos, cell, pbc)
        assert abs(res["energy"][k] - r["energy"]) / len(types) < 2e-6, name
        assert np.abs(res["forces"][at:at + len(types)] - r["forces"]).max() < 2e-5 * max(1.0, np.abs(r["forces"]).max()), name
        at += len(types)
    p = modelgen3l.write_model_3l(str(tmp_path / "l3.npz"), elements=("Al", "Ni", "Ti"), lmax=3, channels=(32, 16, 32), rho_width=24,
                                  embedding=12, radial_hidden=48, seed=5)
    ref = refcpu.RefModel(p, ["Ni", "Ti", "Al"])
    sysm = backend.System(backend.Model(p), ["Ni", "Ti", "Al"])
    rng = np.random.default_rng(2)
    name, types, pos, cell, pbc = cells[0]
    types = rng.integers(1, 4, len(types)).astype(np.int32)
    r, g = ref.compute(types, pos, cell, pbc), sysm.compute(types, pos, cell, pbc)
    assert abs(g["energy"] - r["energy"]) / len(types) < 2e-6
    assert np.abs(g["forces"] - r["forces"]).max() < 2e-5 * max(1.0, np.abs(r["forces"]).max())
    assert np.abs(g["virial"] - r["virial"]).max() < 2e-5 * max(1.0, np.abs(r["virial"]).max())


@pytest.mark.gpu
def test_gpu_tensor_core_operations(backend, small3l, monkeypatch):
    """The projections, reduces and FCs of the layer chains as tensor-core grouped GEMMs (the form large evaluations
    take), forced on a small structure: same results as the SIMT kernels to 3 x tf32 accuracy."""
    name, types, pos, cell, pbc = next(_cells())
    monkeypatch.setenv("GRACE_B200_DENSE", "ops")
    a = backend.System(backend.Model(small3l), ["Al", "Ni"]).compute(types, pos, cell, pbc)
    monkeypatch.setenv("GRACE_B200_DENSE", "tc")
    b = backend.System(backend.Model(small3l), ["Al", "Ni"]).compute(types, pos, cell, pbc)
    assert abs(a["energy"] - b["energy"]) / len(types) < 1e-6
    assert np.abs(a["forces"] - b["forces"]).max() < 2e-5 * max(1.0, np.abs(a["forces"]).max())


@pytest.mark.gpu
def test_gpu_forward_bond_sums_on_tensor_cores(backend, small3l, tmp_path, monkeypatch):
    """GRACE_B200_3L_MMA=1: the forward bond sums as mma.sync tf32 matrix products (three instructions per product on
    hi / lo splits) instead of the register-tile kernel: same energies."""
    from oracle import refcpu
    if not refcpu.available():
        pytest.skip("oracle/_ref is not built")
    monkeypatch.setenv("GRACE_B200_3L_MMA", "1")
    p = modelgen3l.write_model_3l(str(tmp_path / "l4.npz"), elements=("Al", "Ni"), lmax=4, channels=(32, 16, 32), rho_width=16,
                                  embedding=8, radial_hidden=32, seed=9)
    for path in (small3l, p):
        ref = refcpu.RefModel(path, ["Al", "Ni"])
        sysm = backend.System(backend.Model(path), ["Al", "Ni"])
        for name, types, pos, cell, pbc in list(_cells())[:3]:
            r, g = ref.compute(types, pos, cell, pbc), sysm.compute(types, pos, cell, pbc, energies=True)
            assert np.abs(g["energies"] - r["energies"]).max() < 5e-6, name
            assert np.abs(g["forces"] - r["forces"]).max() < 2e-5 * max(1.0, np.abs(r["forces"]).max()), name


@pytest.mark.gpu
def test_gpu_passes_over_atom_chunks(backend, small3l, monkeypatch):
    """GRACE_B200_3L_CHUNK: every layer in passes of at most that many atoms through one arena, the reverse pass
    recomputing the forward tensors of a chunk (what structures too large to keep all tensors get): same results as
    the single pass that keeps them."""
    name, types, pos, cell, pbc = next(_cells())
    sysm = backend.System(backend.Model(small3l), ["Al", "Ni"])
    a = sysm.compute(types, pos, cell, pbc, energies=True)
    monkeypatch.setenv("GRACE_B200_3L_CHUNK", "12")      # 32 atoms: passes of 12, 12 and 8
    b = sysm.compute(types, pos, cell, pbc, energies=True)
    assert np.abs(a["energies"] - b["energies"]).max() < 1e-6
    assert np.abs(a["forces"] - b["forces"]).max() < 2e-5 * max(1.0, np.abs(a["forces"]).max())
    assert np.abs(a["virial"] - b["virial"]).max() < 2e-5 * max(1.0, np.abs(a["virial"]).max())
