"""Test double for thundersvm_b200.sharded: the numerical steps done on the CPU with the oracle, so
that the multi-rank host logic (ownership, exchange, merge, buffer rotation, termination) can run
under the gloo backend without a GPU. Used by tests only."""
import numpy as np
import torch

from oracle import port_binding as P


class OracleOps:
    device = torch.device("cpu")

    class _KM:
        pass

    def kernel_matrix(self, X_local, kernel, gamma, coef0, degree):
        km = self._KM()
        km.X = P.Csr(dense=X_local.numpy())
        km.kw = dict(kernel=kernel, gamma=gamma, coef0=coef0, degree=degree)
        return km

    def self_dot(self, km):
        return torch.from_numpy(P.self_dot(km.X))

    def diag(self, km):
        return torch.from_numpy(P.diag(km.X, **km.kw))

    def selector(self, n_local, ws):
        return None

    @staticmethod
    def _lists(solver):
        if solver == "c":
            return [(None, "up", True), (None, "low", False)]
        return [(1, "up", True), (-1, "up", True), (1, "low", False), (-1, "low", False)]

    def candidates(self, sel, f, alpha, y, Cp, Cn, want, in_ws, solver, id_offset):
        f, a, y = f.numpy(), alpha.numpy(), y.numpy()
        n = len(f)
        free_slot = np.ones(n, bool) if in_ws is None else in_ws.numpy()[:n] == 0
        up = ((y > 0) & (a < Cp)) | ((y < 0) & (a > 0))
        low = ((y > 0) & (a > 0)) | ((y < 0) & (a < Cn))
        cf = np.zeros((len(self._lists(solver)), want))
        ci = np.full((len(self._lists(solver)), want), -1, np.int32)
        for l, (cls, which, asc) in enumerate(self._lists(solver)):
            ok = free_slot & (up if which == "up" else low)
            if cls is not None:
                ok &= (y > 0) if cls > 0 else (y < 0)
            idx = np.nonzero(ok)[0]
            order = np.lexsort((idx, f[idx]))
            idx = idx[order] if asc else idx[order][::-1]
            idx = idx[:want]
            cf[l, :len(idx)] = f[idx]
            ci[l, :len(idx)] = idx + id_offset
        return torch.from_numpy(cf), torch.from_numpy(ci)

    def merge(self, sel, cand_f, cand_id, want, solver):
        cf, ci = cand_f.numpy(), cand_id.numpy()
        lists = []
        for l, (_, _, asc) in enumerate(self._lists(solver)):
            ok = ci[l] >= 0
            f, i = cf[l][ok], ci[l][ok]
            order = np.lexsort((i, f))
            i = i[order] if asc else i[order][::-1]
            lists.append(list(i[:want]))
        taken, out, ptr = set(), [], [0] * len(lists)
        progressed = True
        while len(out) < want and progressed:
            progressed = False
            for l, lst in enumerate(lists):
                if len(out) >= want:
                    break
                while ptr[l] < len(lst) and lst[ptr[l]] in taken:
                    ptr[l] += 1
                if ptr[l] < len(lst):
                    out.append(lst[ptr[l]]); taken.add(lst[ptr[l]]); ptr[l] += 1
                    progressed = True
        out += [-1] * (want - len(out))
        return torch.tensor(out, dtype=torch.int32)

    def rows_for_features(self, km, T, sd_T, out):
        K = P.kernel_rows_ins(km.X, P.Csr(dense=T.numpy()), **km.kw)
        out[:, :K.shape[1]] = torch.from_numpy(K)
        return out

    def local_smo(self, kww, diag_ws, y_ws, f_ws, alpha_ws, Cp, Cn, eps, max_iter, solver):
        ws = kww.shape[0]
        kind = "c" if solver == "c" else "nu"
        a, ad, diff = P.local_smo(kind, y_ws.numpy(), f_ws.numpy(), alpha_ws.numpy(), np.arange(ws, dtype=np.int32), Cp,
                                  Cn, kww.numpy(), diag_ws.numpy(), eps, max_iter=max_iter, cuda_semantics=1)
        return torch.from_numpy(a), torch.from_numpy(ad), torch.from_numpy(diff)

    def update_f(self, f, alpha_diff, rows):
        n = f.numel()
        new = P.update_f(f.numpy(), alpha_diff.numpy(), np.ascontiguousarray(rows.numpy()[:, :n]))
        f.copy_(torch.from_numpy(new))
        return f

    def rho_partials(self, f, alpha, y, Cp, Cn):
        f, a, y = f.numpy(), alpha.numpy(), y.numpy()
        up = ((y > 0) & (a < Cp)) | ((y < 0) & (a > 0))
        low = ((y > 0) & (a > 0)) | ((y < 0) & (a < Cn))
        p, ng = y > 0, y < 0
        fp, fn = p & (a > 0) & (a < Cp), ng & (a > 0) & (a < Cn)

        def mn(mask):
            return f[mask].min() if mask.any() else np.inf

        def mx(mask):
            return f[mask].max() if mask.any() else -np.inf

        out = [fp.sum(), f[fp].sum(), fn.sum(), f[fn].sum(), (a - (f + y) * a * y / 2).sum(), mn(up & p), mx(low & p),
               mn(up & ng), mx(low & ng), mx(up & p), mn(low & p), mx(up & ng), mn(low & ng)]
        return torch.tensor(out, dtype=torch.float64)

    def solve_pair(self, X_pair, y, C, eps, ws, kernel, gamma, coef0, degree):
        X = P.Csr(dense=X_pair.numpy())
        yy = y.numpy().astype(np.int32)
        r = P.smo_solve(X, yy, np.zeros(len(yy)), -yy.astype(np.float64), eps, C, C, ws, kernel=kernel, gamma=gamma,
                        coef0=coef0, degree=degree)
        return torch.from_numpy(r["alpha"]), float(r["rho"])

    def predict_labels(self, sv, coef, n_sv, rho, n_classes, T, kernel, gamma, coef0, degree):
        dec = P.predict_dec(P.Csr(dense=sv.numpy()), np.ascontiguousarray(coef), np.asarray(n_sv, np.int32),
                            np.asarray(rho, np.float64), n_classes, P.Csr(dense=T.numpy()), kernel=kernel, gamma=gamma,
                            coef0=coef0, degree=degree)
        return torch.from_numpy(P.vote(dec, n_classes).astype(np.int32))

