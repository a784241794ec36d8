"""Slab domain decomposition of one structure over the GPUs of a node, one process per GPU.

Every atom's energy depends on the atoms within `layers x cutoff` of it, so the structure shards by atoms: rank r owns
the atoms of one slab of the cell and evaluates them together with a halo of ghost atoms (copies of atoms other ranks
own, periodic images included) as a sub-system that is open along the slab axis and keeps the cell's other two
directions.  The library leaves the ghosts' own energies out (`System.set_owned`), so the forces it returns are the
gradient of the owned energies with respect to every atom of the sub-system; the ghost rows go back to their owners
(one all-to-all of force rows, whose blocks also carry each rank's energy and virial, so the totals need no second
collective).  This is the
"halo = layers x cutoff, one return" scheme; the reference's own multi-GPU runs go through LAMMPS' ghost atoms and
forward / reverse communication (libgrace/include/grace/system.h:56-60, libgrace/include/grace/kk/grace_2l_kk.h:136-153).

The plan is plain numpy and is computed by every rank for all ranks from the replicated structure (no communication at
set-up); only `DistributedSystem.step` talks to other ranks.  With the CUDA library the exchange runs inside the
library's compute call on its own stream (NCCL send / receive pairs, `backend.System.set_exchange`); the torch.distributed
exchange below serves engines injected for tests (CPU, gloo)."""
import numpy as np


def slab_axis(cell, pbc):
    """The cell direction with the largest perpendicular height (slabs are cut across it)."""
    cell = np.asarray(cell, dtype=np.float64)
    vol = abs(np.linalg.det(cell))
    heights = [vol / np.linalg.norm(np.cross(cell[(k + 1) % 3], cell[(k + 2) % 3])) for k in range(3)]
    return int(np.argmax(heights)), heights


class SlabPlan:
    """owned[r]: indices of the atoms rank r owns; ghost_atom[r], ghost_shift[r]: the ghosts of rank r as (atom index,
    integer image along the slab axis), ordered by owner rank; ghost_owner[r]: that owner."""

    def __init__(self, positions, cell, pbc, world, halo, inner=None):
        """halo: width of the ghost shell around a slab; inner: width of the part of it whose atoms owned atoms have
        as neighbours (cutoff + skin; default: the whole halo).  A model of one layer needs halo = inner."""
        positions = np.asarray(positions, dtype=np.float64)
        self.cell = np.asarray(cell, dtype=np.float64).reshape(3, 3)
        self.pbc = np.asarray(pbc).astype(bool).reshape(3)
        self.world = int(world)
        self.n = len(positions)
        self.axis, heights = slab_axis(self.cell, self.pbc)
        ax = self.axis
        f = positions @ np.linalg.inv(self.cell)[:, ax]
        periodic = bool(self.pbc[ax])
        if periodic:
            self.wrap = np.floor(f).astype(np.int64)      # image removed from each atom along the axis
            f = f - self.wrap
            lo0, span = 0.0, 1.0
        else:
            self.wrap = np.zeros(self.n, dtype=np.int64)
            lo0 = float(f.min()) if self.n else 0.0
            span = max(float(f.max()) - lo0, 1e-9) * (1.0 + 1e-12) if self.n else 1.0
        self.frac = f
        owner = np.clip(np.floor((f - lo0) / span * world).astype(np.int64), 0, world - 1)
        self.owner = owner
        hf = halo / heights[ax]                            # halo in fractional units of the axis
        hin = (halo if inner is None else min(inner, halo)) / heights[ax]
        self.owned, self.ghost_atom, self.ghost_shift, self.ghost_owner, self.n_inner = [], [], [], [], []
        self.sub_pbc = self.pbc.copy()
        if world > 1:
            self.sub_pbc[ax] = False
        # the library sorts atoms by cell-list bin with the first cell vector slowest: with the slab axis first, owned
        # atoms, inner ghosts and outer ghosts are runs of its order (cyclic rotation: handedness kept)
        self.sub_cell = np.roll(self.cell, -ax, axis=0)
        self.sub_pbc = np.roll(self.sub_pbc, -ax)
        for r in range(world):
            own = np.nonzero(owner == r)[0]
            self.owned.append(own)
            if world == 1:
                self.ghost_atom.append(np.zeros(0, np.int64)); self.ghost_shift.append(np.zeros(0, np.int64))
                self.ghost_owner.append(np.zeros(0, np.int64)); self.n_inner.append(0)
                continue
            lo, hi = lo0 + span * r / world, lo0 + span * (r + 1) / world
            ga, gs, outer = [], [], []
            smax = int(np.ceil(hf)) + 1 if periodic else 0
            for s in range(-smax, smax + 1):
                g = f + s
                m = (g >= lo - hf) & (g < hi + hf)
                if s == 0:
                    m &= owner != r
                idx = np.nonzero(m)[0]
                ga.append(idx); gs.append(np.full(len(idx), s, dtype=np.int64))
                outer.append(((g[idx] < lo - hin) | (g[idx] >= hi + hin)).astype(np.int64))
            ga, gs, outer = np.concatenate(ga), np.concatenate(gs), np.concatenate(outer)
            order = np.lexsort((gs, ga, owner[ga], outer))  # inner ghosts first; then by owner, atom, image
            self.ghost_atom.append(ga[order]); self.ghost_shift.append(gs[order])
            self.ghost_owner.append(owner[ga[order]])
            self.n_inner.append(int(np.sum(outer == 0)))
        # where each owned atom sits in its owner's sub-system
        self.local_index = np.zeros(self.n, dtype=np.int64)
        for r in range(world):
            self.local_index[self.owned[r]] = np.arange(len(self.owned[r]))

    def subsystem(self, rank, types, positions):
        """(types, positions, nlocal) of rank's sub-system: owned atoms first, then its ghosts at their image positions."""
        types = np.asarray(types)
        positions = np.asarray(positions, dtype=np.float64)
        own, ga, gs = self.owned[rank], self.ghost_atom[rank], self.ghost_shift[rank]
        a = self.cell[self.axis]
        if self.world == 1:
            return types[own].astype(np.int32), np.ascontiguousarray(positions[own]), len(own)
        p_own = positions[own] - self.wrap[own, None] * a
        p_gh = positions[ga] + (gs - self.wrap[ga])[:, None] * a
        return (np.concatenate([types[own], types[ga]]).astype(np.int32),
                np.ascontiguousarray(np.concatenate([p_own, p_gh])), len(own))

    def send_order(self, rank):
        """the ghosts of rank (positions in its ghost list) grouped by owner: the order its force rows are sent in"""
        return np.argsort(self.ghost_owner[rank], kind="stable")

    def send_counts(self, rank):
        """ghost rows rank sends back to each owner"""
        return np.bincount(self.ghost_owner[rank], minlength=self.world).astype(np.int64)

    def recv_counts(self, rank):
        return np.array([int(np.sum(self.ghost_owner[r] == rank)) for r in range(self.world)], dtype=np.int64)

    def recv_index(self, rank):
        """local index (in rank's owned atoms) of every row it receives, in the order the senders' rows arrive"""
        parts = []
        for r in range(self.world):
            o = self.send_order(r)
            parts.append(self.local_index[self.ghost_atom[r][o][self.ghost_owner[r][o] == rank]])
        return np.concatenate(parts) if parts else np.zeros(0, np.int64)

    def assemble(self, per_rank_forces):
        """Single-process stand-in for the exchange: forces [n, 3] of the whole structure from every rank's
        sub-system forces (owned rows, then ghost rows)."""
        out = np.zeros((self.n, 3))
        for r in range(self.world):
            f = np.asarray(per_rank_forces[r])
            nl = len(self.owned[r])
            np.add.at(out, self.owned[r], f[:nl])
            np.add.at(out, self.ghost_atom[r], f[nl:])
        return out


def halo_width(layers, cutoff, skin):
    """Ghosts needed by the owned energies: `layers` hops of at most cutoff, each allowed to shrink by the Verlet
    skin before the neighbour list is rebuilt."""
    return layers * (cutoff + skin)


def make_plan(positions, cell, pbc, world, layers, cutoff, skin):
    """the plan of a model with `layers` message-passing layers"""
    return SlabPlan(positions, cell, pbc, world, halo_width(layers, cutoff, skin),
                    inner=halo_width(1, cutoff, skin) if layers > 1 else None)


def init_library_comm(rank, world):
    """Creates the library's NCCL communicator of a torch.distributed job: rank 0's unique id goes round through the
    job's default process group."""
    import torch.distributed as dist
    from . import backend as B
    ids = [B.comm_unique_id() if rank == 0 else None]
    dist.broadcast_object_list(ids, src=0)
    B.comm_init(ids[0], rank, world)


class DistributedSystem:
    """One rank's part of a decomposed structure on its GPU: `step()` evaluates the sub-system through the C ABI
    (device pointers); the library returns ghost forces to their owners and sums energy and virial over its
    communicator inside that call (`init_library_comm` first).  `compute(positions, ...)` callables other than the CUDA
    library can be injected for tests (`engine=`): their exchange goes through torch.distributed."""

    def __init__(self, plan, rank, types, positions, species=None, model=None, skin=0.5, chunksize=-1, device=None,
                 engine=None, group=None):
        import torch
        self.torch = torch
        self.plan, self.rank, self.group = plan, rank, group
        self.types, self.pos, self.nlocal = plan.subsystem(rank, types, positions)
        self.n = len(self.types)
        self.device = device if device is not None else torch.device("cpu")
        # every block of the all-to-all carries the ghost rows for that owner and 3 more rows with this rank's energy and
        # virial (9 doubles, 7 used), so that one collective both returns the forces and sums the totals
        W = plan.world
        sc, rc = plan.send_counts(rank), plan.recv_counts(rank)
        self.send_splits = [int(c) + 3 for c in sc]
        self.recv_splits = [int(c) + 3 for c in rc]
        n = self.n
        order = plan.send_order(rank) + self.nlocal
        send_idx, at = [], 0
        for d in range(W):
            send_idx.append(order[at:at + int(sc[d])]); at += int(sc[d])
            send_idx.append(np.array([n, n + 1, n + 2], dtype=np.int64))          # the rows behind the forces: energy, virial
        self.send_idx = torch.from_numpy(np.concatenate(send_idx)).to(self.device)
        ridx, recv_idx, at = plan.recv_index(rank), [], 0
        for r in range(W):
            recv_idx.append(ridx[at:at + int(rc[r])]); at += int(rc[r])
            # the totals of the other ranks add onto this rank's own rows; its own copy goes to a scratch row
            recv_idx.append(np.array([n, n + 1, n + 2] if r != rank else [n + 3, n + 3, n + 3], dtype=np.int64))
        self.recv_idx = torch.from_numpy(np.concatenate(recv_idx)).to(self.device)
        self.layers = 1
        self.engine = engine
        self.library_exchange = False
        if engine is None:
            from . import backend as B
            self.system = B.System(model, species, skin=skin, chunksize=chunksize)
            self.layers = model.layers
            if plan.world > 1:     # one layer: no ghost needs anything but its position
                ninner = self.nlocal + (plan.n_inner[rank] if self.layers > 1 else 0)
                if B.comm_size() == plan.world:
                    self.system.set_exchange(self.n, self.nlocal, ninner, sc, order, rc, plan.recv_index(rank))
                    self.library_exchange = True
                else:      # no library communicator (single-process checks): owned / ghost split only
                    self.system.set_owned(self.nlocal, ninner)
        dev = self.device
        self.d_types = torch.from_numpy(self.types).to(dev)
        self.d_pos = torch.from_numpy(self.pos).to(dev)
        # forces [n, 3], then 3 rows holding energy and virial[6] (and 2 unused doubles), then a scratch row
        self.d_fx = torch.zeros((self.n + 4, 3), dtype=torch.float64, device=dev)
        self.d_f = self.d_fx[:max(self.n, 1)]
        self.d_ev = self.d_fx.view(-1)[3 * self.n:3 * self.n + 7]
        self.d_recv = torch.zeros((sum(self.recv_splits), 3), dtype=torch.float64, device=dev)

    def load_positions(self, sub_positions_pinned):
        """host -> device copy of this rank's sub-system positions (the end-to-end leg)"""
        self.d_pos.copy_(sub_positions_pinned, non_blocking=True)

    def evaluate_local(self):
        """the sub-system through the library (or the injected engine): fills d_ev and d_f"""
        if self.engine is not None:
            e, v, f = self.engine(self.types, self.d_pos.cpu().numpy(), self.plan.sub_cell, self.plan.sub_pbc,
                                  self.nlocal)
            self.d_ev.copy_(self.torch.from_numpy(np.concatenate([[e], v])))
            if self.n:
                self.d_f[:self.n].copy_(self.torch.from_numpy(np.asarray(f)))
            return
        ev = self.d_ev.data_ptr()
        self.system.compute_device(self.d_types.data_ptr(), self.d_pos.data_ptr(), self.plan.sub_cell,
                                   self.plan.sub_pbc, ev, forces=self.d_f.data_ptr(), virial=ev + 8, n=self.n)

    def exchange(self):
        """ghost forces back to their owners, energy and virial summed over the ranks"""
        import torch.distributed as dist
        torch = self.torch
        if self.plan.world == 1 or self.library_exchange:
            return
        self.d_fx.view(-1)[3 * self.n + 7:3 * self.n + 12].zero_()    # the unused doubles of the total rows, the scratch row
        send = self.d_fx.index_select(0, self.send_idx)
        dist.all_to_all_single(self.d_recv, send, self.recv_splits, self.send_splits, group=self.group)
        self.d_fx.index_add_(0, self.recv_idx, self.d_recv)

    def step(self):
        self.evaluate_local()
        self.exchange()

    @property
    def energy(self):
        return float(self.d_ev[0].item())

    @property
    def virial(self):
        return self.d_ev[1:].cpu().numpy()

    @property
    def owned_forces(self):
        return self.d_f[:self.nlocal]
