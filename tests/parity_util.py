"""Sampled-column parity of a full-size aggregation step against the CPU checker.

A column's aggregate depends on that column alone (its K gradients, its K residuals, its owner's stripe residual), so
the CPU checker can replay any sample of columns of a tensor that is far too large to replay whole
(oracle.exchange.aggregate_columns).  This module captures, for a seeded sample of columns of every tensor, what goes
into one step (gradient, residual and stripe residual columns) and what comes out of it (aggregate, new residual, new
stripe residual, gathered packed column), and compares the outputs with the replay, bit for bit.

Used by the GPU tests on in-process rank groups and by bench.py on real multi-GPU runs (one process per GPU), where
the ranks' inputs are all-gathered first.  Test infrastructure: the product never imports it.
"""
import numpy as np
import torch

from oracle import exchange


def pick_columns(shapes, K, seed, per_tensor=24):
    """Seeded sample of columns per tensor: random ones plus the first and last column of the matrix and of two stripes."""
    rng = np.random.default_rng(seed)
    cols = []
    for (M, N) in shapes:
        if M == 0 or N == 0:
            cols.append([])
            continue
        c = set(int(x) for x in rng.integers(0, N, size=min(per_tensor, N))) | {0, N - 1}
        for p in {int(x) for x in rng.integers(0, K, size=2)}:
            s, n = exchange.stripe(N, p, K)
            if n:
                c |= {s, s + n - 1}
        cols.append(sorted(c))
    return cols


class RankCapture:
    """What one rank contributes to, and gets out of, the checked step, for the sampled columns."""

    def __init__(self, lib, agg, rank, K, shapes, bits, cols):
        self.lib, self.agg, self.rank, self.K, self.shapes, self.bits, self.cols = lib, agg, rank, K, shapes, bits, cols
        self.inp = None
        self.out = None

    def _res_cols(self, i, dev):
        M, N = self.shapes[i]
        buf = torch.empty((N, M), dtype=torch.float32, device=dev)
        self.agg.copy_residual(i, 0, buf.data_ptr())
        torch.cuda.synchronize(dev)
        return buf[torch.tensor(self.cols[i], device=dev)].cpu().numpy()

    def _sres_cols(self, i, dev):
        """(n, M) for all sampled columns; rows of columns this rank does not own stay zero."""
        M, N = self.shapes[i]
        out = np.zeros((len(self.cols[i]), M), np.float32)
        s, n = exchange.stripe(N, self.rank, self.K)
        mine = [(k, c) for k, c in enumerate(self.cols[i]) if s <= c < s + n]
        if self.K > 1 and n and mine:
            buf = torch.empty((n, M), dtype=torch.float32, device=dev)
            self.agg.copy_residual(i, 1, buf.data_ptr())
            torch.cuda.synchronize(dev)
            rows = buf[torch.tensor([c - s for _, c in mine], device=dev)].cpu().numpy()
            for (k, _), row in zip(mine, rows):
                out[k] = row
        return out

    def before(self, grads):
        """grads: this rank's device gradients, still holding the step's input."""
        dev = grads[0].device
        self.inp = {"g": [], "res": [], "sres": []}
        for i, (M, N) in enumerate(self.shapes):
            if not self.cols[i]:
                for k in self.inp:
                    self.inp[k].append(np.zeros((0, M), np.float32))
                continue
            self.inp["g"].append(grads[i][torch.tensor(self.cols[i], device=dev)].cpu().numpy())
            self.inp["res"].append(self._res_cols(i, dev))
            self.inp["sres"].append(self._sres_cols(i, dev))

    def after(self, grads):
        """grads: this rank's device gradients, now holding the aggregate."""
        dev = grads[0].device
        self.out = {"g": [], "res": [], "sres": [], "pk": []}
        for i, (M, N) in enumerate(self.shapes):
            if not self.cols[i]:
                for k in ("g", "res", "sres"):
                    self.out[k].append(np.zeros((0, M), np.float32))
                self.out["pk"].append(np.zeros((0, 0), np.uint8))
                continue
            idx = torch.tensor(self.cols[i], device=dev)
            self.out["g"].append(grads[i][idx].cpu().numpy())
            self.out["res"].append(self._res_cols(i, dev))
            self.out["sres"].append(self._sres_cols(i, dev))
            C = self.lib.packed_col_bytes(M, self.bits)
            pk = torch.zeros(N * C, dtype=torch.uint8, device=dev)
            self.agg.copy_packed(i, pk.data_ptr())
            torch.cuda.synchronize(dev)
            self.out["pk"].append(pk.view(N, C)[idx].cpu().numpy())

    # ---- the inputs as one flat float32 vector (same length on every rank), for an all-gather -----------------------
    def flat_inputs(self):
        return np.concatenate([a.reshape(-1) for k in ("g", "res", "sres") for a in self.inp[k]] + [np.zeros(1, np.float32)])

    def inputs_from_flat(self, flat):
        inp = {"g": [], "res": [], "sres": []}
        o = 0
        for k in ("g", "res", "sres"):
            for i, (M, N) in enumerate(self.shapes):
                n = len(self.cols[i]) * M
                inp[k].append(flat[o:o + n].reshape(len(self.cols[i]), M).copy())
                o += n
        return inp


def verify(be, me, all_inputs, zero_thr=True, self_quant=True):
    """me: the RankCapture whose outputs are checked; all_inputs[r]: the input dict of rank r (all K of them).
    Returns the number of columns compared; raises AssertionError on the first differing byte."""
    K, shapes, bits, cols = me.K, me.shapes, me.bits, me.cols
    checked = 0
    for i, (M, N) in enumerate(shapes):
        if not cols[i]:
            continue
        owners = [exchange.owner_of(c, N, K) for c in cols[i]]
        for p in sorted(set(owners)):
            idx = [k for k, o in enumerate(owners) if o == p]
            g = [np.ascontiguousarray(all_inputs[r]["g"][i][idx]) for r in range(K)]
            res = [np.ascontiguousarray(all_inputs[r]["res"][i][idx]) for r in range(K)]
            sres = np.ascontiguousarray(all_inputs[p]["sres"][i][idx])
            out, pk = exchange.aggregate_columns(be, p, g, res, sres, bits, zero_thr, self_quant)
            what = f"tensor {i} ({M}x{N}), rank {me.rank}, columns {[cols[i][k] for k in idx][:4]}.. owned by rank {p}"
            assert np.array_equal(me.out["g"][i][idx].view(np.uint32), out.view(np.uint32)), "aggregate differs from the CPU checker: " + what
            assert np.array_equal(me.out["res"][i][idx].view(np.uint32), res[me.rank].view(np.uint32)), "residual differs from the CPU checker: " + what
            C = me.lib.packed_col_bytes(M, bits)
            assert np.array_equal(me.out["pk"][i][idx].reshape(-1), pk.reshape(-1)[:len(idx) * C]), "packed column differs from the CPU checker: " + what
            if p == me.rank and K > 1:
                assert np.array_equal(me.out["sres"][i][idx].view(np.uint32), sres.view(np.uint32)), "stripe residual differs from the CPU checker: " + what
            checked += len(idx)
    return checked
