"""A CPU (numpy + oracle) implementation of the four expert-parallel stages, used only to
test the exchange protocol of ExpertParallelEngine with gloo.  It follows the oracle's
arithmetic, so the expert-parallel result must equal oracle.layer_forward bit for bit."""
import numpy as np
import torch

import __graft_entry__ as entry


def sequential_matvec(a_row: np.ndarray, w: np.ndarray) -> np.ndarray:
    """out[o] = sum_c a[c] * w[o][c] in FP32, c ascending, separate multiply and add."""
    acc = np.zeros(w.shape[0], dtype=np.float32)
    for c in range(w.shape[1]):
        acc = (acc + (a_row[c] * w[:, c]).astype(np.float32)).astype(np.float32)
    return acc


class NumpyStages:
    def __init__(self, ocfg, weights, rank, world):
        self.oracle = entry.load_oracle()
        self.cfg, self.w, self.rank, self.world = ocfg, weights, rank, world
        self.per_rank = ocfg.experts // world
        H = ocfg.hidden
        self.record_bytes = (H // 2 + H // 16 + 12 + 15) // 16 * 16
        o = self.oracle
        self.up = {e: o.dequant_nvfp4(weights.up[e].packed, weights.up[e].scales,
                                      weights.up[e].tensor_scale)
                   for e in range(rank * self.per_rank, (rank + 1) * self.per_rank)}
        self.down = {e: o.dequant_nvfp4(weights.down[e].packed, weights.down[e].scales,
                                        weights.down[e].tensor_scale) for e in self.up}
        self.sup = o.dequant_nvfp4(weights.shared_up.packed, weights.shared_up.scales,
                                   weights.shared_up.tensor_scale)
        self.sdown = o.dequant_nvfp4(weights.shared_down.packed, weights.shared_down.scales,
                                     weights.shared_down.tensor_scale)

    def _ffn(self, a_deq, up, down):
        o = self.oracle
        h = sequential_matvec(a_deq, up)
        h = np.where(h > 0, h * h, 0).astype(np.float32)
        p, s, ts = o.pack_nvfp4(h[None, :])
        return sequential_matvec(o.dequant_nvfp4(p, s, ts)[0], down)

    def count_buffer(self):
        return torch.zeros((self.world,), dtype=torch.int32)

    def dispatch(self, x, capacity=0):
        o, cfg = self.oracle, self.cfg
        xs = x.to(torch.float32).numpy()
        y = o.rmsnorm(xs, self.w.norm_weight, cfg.rms_eps)
        logits = o.router_logits(y, self.w.gate)
        idx, wt = o.select_top_experts(logits, self.w.bias, cfg.top_k, cfg.n_group, cfg.topk_group,
                                       cfg.norm_topk_prob, cfg.routed_scaling)
        self.packed, self.scales, self.ts = o.pack_nvfp4_per_row(y)
        T, K, H = xs.shape[0], cfg.top_k, cfg.hidden
        dest = idx // self.per_rank
        counts = np.bincount(dest.ravel(), minlength=self.world).astype(np.int32)
        if capacity > 0:
            assert counts.max() <= capacity
            offsets = np.arange(self.world) * capacity
            records = np.zeros((self.world * capacity, self.record_bytes), dtype=np.uint8)
        else:
            offsets = np.concatenate([[0], np.cumsum(counts)[:-1]])
            records = np.zeros((T * K, self.record_bytes), dtype=np.uint8)
        cursor = np.zeros(self.world, dtype=np.int64)
        self.position = np.zeros((T, K), dtype=np.int64)
        for t in range(T):
            for k in range(K):
                r = dest[t, k]
                pos = offsets[r] + cursor[r]
                cursor[r] += 1
                rec = records[pos]
                rec[:H // 2] = self.packed[t]
                rec[H // 2:H // 2 + H // 16] = self.scales[t]
                tail = H // 2 + H // 16
                rec[tail:tail + 4] = np.frombuffer(np.float32(self.ts[t]).tobytes(), np.uint8)
                rec[tail + 4:tail + 8] = np.frombuffer(np.float32(wt[t, k]).tobytes(), np.uint8)
                rec[tail + 8:tail + 12] = np.frombuffer(
                    np.int32(idx[t, k] - r * self.per_rank).tobytes(), np.uint8)
                self.position[t, k] = pos
        return torch.from_numpy(records), torch.from_numpy(counts)

    # no streams on the CPU: the hooks of the device implementation are no-ops here
    def comm_stream(self):
        import contextlib
        return contextlib.nullcontext()

    def main_to_comm(self):
        pass

    def comm_to_main(self):
        pass

    def experts(self, recv, count, row_offset=0, valid_counts=None, capacity=0):
        o, H = self.oracle, self.cfg.hidden
        recs = recv.numpy()
        out = np.zeros((count, H), dtype=np.float32)
        tail = H // 2 + H // 16
        for i in range(count):
            if valid_counts is not None and (i % capacity) >= int(valid_counts[i // capacity]):
                continue
            rec = recs[i]
            ts = rec[tail:tail + 4].copy().view(np.float32)[0]
            weight = rec[tail + 4:tail + 8].copy().view(np.float32)[0]
            local = int(rec[tail + 8:tail + 12].copy().view(np.int32)[0])
            e = self.rank * self.per_rank + local
            a = o.dequant_nvfp4(rec[None, :H // 2], rec[None, H // 2:tail], float(ts))[0]
            out[i] = (self._ffn(a, self.up[e], self.down[e]) * weight).astype(np.float32)
        return torch.from_numpy(out)

    def shared(self):
        o = self.oracle
        T = self.packed.shape[0]
        self.shared_rows = np.stack([
            self._ffn(o.dequant_nvfp4(self.packed[t:t + 1], self.scales[t:t + 1],
                                      float(self.ts[t]))[0], self.sup, self.sdown)
            for t in range(T)])

    def combine(self, x, back, out):
        rows = back.numpy()
        xs = x.to(torch.float32).numpy()
        T, K = self.position.shape
        for t in range(T):
            routed = rows[self.position[t, 0]].copy()
            for k in range(1, K):
                routed = (routed + rows[self.position[t, k]]).astype(np.float32)
            mixer = (routed + self.shared_rows[t]).astype(np.float32)
            out[t] = torch.from_numpy((xs[t] + mixer).astype(np.float32))

    def recv_buffer(self, count):
        return torch.empty((count, self.record_bytes), dtype=torch.uint8)

    def back_buffer(self, count):
        return torch.empty((count, self.cfg.hidden), dtype=torch.float32)
