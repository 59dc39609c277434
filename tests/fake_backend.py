"""A stand-in for liblce_b200 that computes each per-chunk call with the float64 oracle on the CPU.

Only used by the CPU tests of the HOST logic (chunk loop, autograd plumbing, vocabulary sharding over
gloo); it mirrors the methods of ``ops.NativeBackend`` one for one.
"""
import numpy as np
import torch

from oracle import oracle


class FakeBackend:
    name = "oracle-fake"
    requires_cuda = False

    def __init__(self):
        self.state = {}
        self.calls = []

    def workspace_bytes(self, prob):
        return 256

    def begin(self, prob, y, workspace):
        self.calls.append("begin")
        self.state[workspace.data_ptr()] = dict(
            n_valid=float((y != prob.ignore_index).sum()), nll=0.0, lse2=0.0, ent=0.0, norm=0.0, zmax=-np.inf,
        )

    def forward_chunk(self, prob, x, At, y, row0, rows, workspace, row_parts):
        self.calls.append("forward_chunk")
        st = self.state[workspace.data_ptr()]
        z = oracle.logits64(x[row0:row0 + rows], At, prob.logit_scale)
        yy = y[row0:row0 + rows].numpy()
        parts = oracle.row_partials(z, yy, prob.vocab_offset, prob.ignore_index)
        local0 = row0 % prob.chunk_rows
        rp = row_parts.view(6, prob.chunk_rows)
        rp[:, local0:local0 + rows] = torch.from_numpy(parts).float()
        st.setdefault("z", {})[row0] = z

    def combine_chunk(self, prob, row_parts_all, y, row0, rows, workspace):
        self.calls.append("combine_chunk")
        st = self.state[workspace.data_ptr()]
        local0 = row0 % prob.chunk_rows
        parts = row_parts_all.view(prob.world, 6, prob.chunk_rows)[:, :, local0:local0 + rows].double().numpy()
        lse, t, ent, q, m = oracle.combine_partials(parts)
        v = (y[row0:row0 + rows] != prob.ignore_index).numpy()
        st["nll"] += float(((lse - t) * v).sum())
        st["lse2"] += float((lse * lse * v).sum())
        st["ent"] += float((ent * v).sum())
        st["norm"] += float(np.sqrt(q).sum())
        st["zmax"] = max(st["zmax"], float(m.max()))
        st.setdefault("lse", {})[row0] = lse

    # The row-partials exchange over peer memory, for one rank: slots keyed by epoch in the table object.
    def parts_bytes(self, prob):
        return 4096

    def parts_push(self, prob, row_parts, row0, rows, table, epoch, stream_of):
        self.calls.append(("parts_push", epoch))
        assert len(table.slots) < 4, "four slots: at most four epochs may be unmerged"
        table.slots[epoch] = row_parts.clone()

    def combine_chunk_peer(self, prob, table, epoch, y, row0, rows, workspace, wait_ms=0):
        self.calls.append(("combine_chunk_peer", epoch))
        self.combine_chunk(prob, table.slots.pop(epoch), y, row0, rows, workspace)
        self.calls.pop()  # the inner combine_chunk entry

    def dz_chunk(self, prob, x, y, row0, rows, workspace):
        self.calls.append("dz_chunk")
        st = self.state[workspace.data_ptr()]
        z, lse = st["z"].pop(row0), st["lse"].pop(row0)
        yy = y[row0:row0 + rows].numpy()
        v = yy != prob.ignore_index
        p = np.exp(z - lse[:, None]) * (1.0 + 2.0 * prob.z_regularization * lse)[:, None]
        yl = yy - prob.vocab_offset
        own = v & (yl >= 0) & (yl < z.shape[1])
        p[np.nonzero(own)[0], yl[own]] -= 1.0
        p *= v[:, None]
        st.setdefault("dz", {})[row0] = p

    def dx_chunk(self, prob, At, row0, rows, workspace, dx):
        self.calls.append("dx_chunk")
        st = self.state[workspace.data_ptr()]
        coef = prob.logit_scale / st["n_valid"]
        dx[row0:row0 + rows] = torch.from_numpy(st["dz"][row0] @ At.double().numpy().T * coef).to(dx.dtype)

    # The dx exchange over peer memory, for one rank: the "exchange buffer" is a dict keyed by epoch.
    def peer_bytes(self, prob, dx_dtype):
        return 4096

    def dx_chunk_peer(self, prob, At, row0, rows, workspace, table, dx_dtype, epoch):
        self.calls.append(("dx_chunk_peer", epoch))
        st = self.state[workspace.data_ptr()]
        coef = prob.logit_scale / st["n_valid"]
        assert epoch not in table.scattered and len(table.scattered) < 2, "at most two epochs in flight"
        table.scattered[epoch] = torch.from_numpy(st["dz"][row0] @ At.double().numpy().T * coef)

    def dx_reduce_peer(self, prob, row0, rows, workspace, table, dx_dtype, epoch, wait_ms=0):
        self.calls.append(("dx_reduce_peer", epoch))
        table.reduced[epoch] = table.scattered[epoch].to(dx_dtype)

    def dx_finish_peer(self, prob, row0, rows, workspace, table, epoch, dx, wait_ms=0):
        self.calls.append(("dx_finish_peer", epoch))
        dx[row0:row0 + rows] = table.reduced.pop(epoch)
        del table.scattered[epoch]

    def dw_chunk(self, prob, x, row0, rows, workspace, dW, dW_res, first, last):
        self.calls.append("dw_chunk")
        st = self.state[workspace.data_ptr()]
        coef = prob.logit_scale / st["n_valid"]
        keys = sorted(k for k in st["dz"] if row0 <= k < row0 + rows)
        dz = np.concatenate([st["dz"].pop(k) for k in keys])
        assert dz.shape[0] == rows
        total = torch.from_numpy(x[row0:row0 + rows].double().numpy().T @ dz * coef)
        if not first:  # the running sum is dW + dW_res (the residual only exists for 16-bit types)
            total = total + dW.double() + (dW_res.double() if dW_res is not None else 0)
        dW.copy_(total.to(dW.dtype))
        if dW_res is not None and not last:
            dW_res.copy_((total - dW.double()).to(dW.dtype))
        assert dW_res is not None or dW.dtype == torch.float32 or (first and last)

    def finalize(self, prob, workspace, out5):
        self.calls.append("finalize")
        st = self.state.pop(workspace.data_ptr())
        R = st["n_valid"]
        with np.errstate(invalid="ignore", divide="ignore"):
            vals = [
                np.float64(st["nll"] + prob.z_regularization * st["lse2"]) / R, np.float64(st["lse2"]) / R,
                st["zmax"], np.float64(st["ent"]) / R, st["norm"] / prob.n_rows_total,
            ]
        out5.copy_(torch.tensor(vals, dtype=torch.float32))

    def grad_scale_cast(self, src, dst, factor):
        self.calls.append("grad_scale_cast")
        dst.copy_((src.double() * factor.double()).to(dst.dtype))

    def read_status(self, workspace):
        return 0
