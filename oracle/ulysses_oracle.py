"""CPU oracle of the fused projection-GEMM + Ulysses all-to-all path.

TEST INFRASTRUCTURE ONLY. Nothing the library ships imports this module; only tests/, the smoke
check and the cpu_baseline / reference arms of bench.py may. It restates, for all P ranks inside
one process, what the reference computes on P GPUs:

  * the unfused Ulysses data flow that the reference's fused kernels are validated against
    (benchmark/reference.py:69-152: per-projection linear, all-to-all, linear backward;
    benchmark/run.py:152-205: full-token FP32 linear, then slice this rank's heads and rows),
  * the Megatron per-head row interleave (benchmark/reference.py:193-203),
  * the padded buffer contents of the fused transport (tests/test_row_blocks.py:115-175:
    head-side buffers [P*cap, H/P] and receive buffers [cap, segments*H]),
  * resize_rank_rows and reduce_bias_grad (fused_gemm_a2a_kernels.py:1086-1188).

Parity pin: checked against outputs of the reference's own unfused modules run under gloo
(tests/golden/make_golden.py produced tests/golden/*.npz from benchmark/reference.py), see
tests/test_oracle_golden.py.

Arithmetic model: inputs are BF16 (or FP32/FP64 for the CPU configuration); every GEMM
accumulates in `acc_dtype` (FP32 by default, FP64 for tight checks) from the exact input values
and is rounded once to the activation dtype, which is what an FP32-accumulating tensor-core GEMM
followed by a BF16 store does up to summation order.
"""
import torch


def interleave_qkv_rows(segment_major, heads, head_dim):
    """Rows in segment-major order [Q; K; V(; G)] -> per-head order [q_h; k_h; v_h(; g_h)].
    Restates benchmark/reference.py:193-203."""
    h = heads * head_dim
    rows = segment_major.shape[0]
    if rows not in (3 * h, 4 * h):
        raise ValueError(f'{rows} rows are not 3 or 4 segments of {h}')
    s = rows // h
    tail = tuple(segment_major.shape[1:])
    return segment_major.reshape((s, heads, head_dim) + tail).transpose(0, 1).reshape(segment_major.shape)


def deinterleave_qkv_rows(per_head, heads, head_dim):
    """Inverse of interleave_qkv_rows."""
    h = heads * head_dim
    s = per_head.shape[0] // h
    tail = tuple(per_head.shape[1:])
    return per_head.reshape((heads, s, head_dim) + tail).transpose(0, 1).reshape(per_head.shape)


def padded_rows(valid, tile):
    """Next multiple of `tile` (fused_gemm_a2a_kernels.py:100-104)."""
    if valid < 1 or tile < 1:
        raise ValueError('Token count and tile height must be positive')
    return -(-valid // tile) * tile


def _mm(a, b, acc_dtype):
    return a.to(acc_dtype) @ b.to(acc_dtype)


class UlyssesOracle:
    """All P ranks of one CP group, simulated on the CPU.

    weight_qkv: [(3+gate)*H, H] in per-head interleaved row order; weight_out: [H, H];
    biases in the same row orders (or None). `dtype` is the activation dtype outputs are rounded to.
    """

    def __init__(self, p, hidden, heads, segments, weight_qkv=None, bias_qkv=None, weight_out=None,
                 bias_out=None, *, dtype=torch.bfloat16, acc_dtype=torch.float32,
                 bias_in_gemm=False, apply_bias=True):
        if heads % p or hidden % heads:
            raise ValueError('heads must split over P and hidden over heads')
        self.p, self.h, self.n, self.s = p, hidden, heads, segments
        self.d = hidden // heads
        self.c = hidden // p  # head-side columns per rank
        self.wq, self.bq, self.wo, self.bo = weight_qkv, bias_qkv, weight_out, bias_out
        self.dtype, self.acc = dtype, acc_dtype
        self.bias_in_gemm, self.apply_bias = bias_in_gemm, apply_bias

    # ------------------------------------------------------------------ QKV projection
    def qkv_sequence_side(self, x):
        """One rank's [M, S*H] projection in weight-row order, rounded to dtype.
        bias_in_gemm adds the bias to the accumulator before rounding
        (fused_gemm_a2a_kernels.py:975-992)."""
        y = _mm(x, self.wq.t(), self.acc)
        if self.bq is not None and self.apply_bias and self.bias_in_gemm:
            y = y + self.bq.to(self.acc)
        return y.to(self.dtype)

    def qkv_forward(self, xs):
        """xs: list of P [M, H]. Returns per destination rank a tuple of `segments` tensors
        [P*M, N/P, D] (rows rank-major). The default bias path is GEMM -> dtype -> + bias -> dtype
        (fused_gemm_a2a_kernels.py:1138-1140)."""
        p, s, d, hpr = self.p, self.s, self.d, self.n // self.p
        m = xs[0].shape[0]
        ys = [self.qkv_sequence_side(x).reshape(m, self.n, s, d) for x in xs]
        outs = []
        for dest in range(p):
            per_seg = []
            for seg in range(s):
                rows = [y[:, dest * hpr:(dest + 1) * hpr, seg, :] for y in ys]
                t = torch.cat(rows, dim=0).contiguous()
                if self.bq is not None and self.apply_bias and not self.bias_in_gemm:
                    b = self.bq.reshape(self.n, s, d)[dest * hpr:(dest + 1) * hpr, seg, :]
                    t = (t.to(self.acc) + b.to(self.acc)).to(self.dtype)
                per_seg.append(t)
            outs.append(tuple(per_seg))
        return outs

    def qkv_heads_buffers(self, xs, capacity):
        """Head-side buffers after the push GEMM and before the ownership copy: per destination a
        list of `segments` [P*capacity, H/P] matrices whose pad rows hold the GEMM of zero rows
        (zero, or the bias when it is added in the GEMM)."""
        p, s, d, hpr = self.p, self.s, self.d, self.n // self.p
        bufs = [[torch.zeros(p * capacity, self.c, dtype=self.dtype) for _ in range(s)] for _ in range(p)]
        for r, x in enumerate(xs):
            xp = torch.zeros(capacity, self.h, dtype=x.dtype)
            xp[:x.shape[0]] = x
            y = self.qkv_sequence_side(xp).reshape(capacity, self.n, s, d)
            for dest in range(p):
                for seg in range(s):
                    bufs[dest][seg][r * capacity:(r + 1) * capacity] = \
                        y[:, dest * hpr:(dest + 1) * hpr, seg, :].reshape(capacity, self.c)
        return bufs

    def qkv_recv_buffer(self, grads, rank, capacity=None):
        """dY of one rank in weight-row column order [rows, S*H]: column block
        ((head*S + seg)*D) of row i holds grads[dest][seg][rank*M + i, head_local, :]
        (fused_gemm_a2a_kernels.py:330-342). grads: per rank a tuple of `segments` [P*M, N/P, D].
        With `capacity`, rows beyond M are exact zeros."""
        p, s, d, hpr = self.p, self.s, self.d, self.n // self.p
        m = grads[0][0].shape[0] // p
        rows = m if capacity is None else capacity
        out = torch.zeros(rows, self.n, s, d, dtype=grads[0][0].dtype)
        for dest in range(p):
            for seg in range(s):
                out[:m, dest * hpr:(dest + 1) * hpr, seg, :] = grads[dest][seg][rank * m:(rank + 1) * m]
        return out.reshape(rows, s * self.h)

    def qkv_backward(self, xs, grads):
        """Returns per rank (dx [M,H] in dtype, dW [S*H,H] and dbias [S*H] in acc dtype, both
        rank-local partial sums in interleaved row order)."""
        res = []
        for r, x in enumerate(xs):
            dy = self.qkv_recv_buffer(grads, r)
            dx = _mm(dy, self.wq, self.acc).to(self.dtype)
            dw = _mm(dy.t(), x, self.acc)
            db = dy.to(self.acc).sum(0)
            res.append((dx, dw, db))
        return res

    # ------------------------------------------------------------------ output projection
    def out_recv_buffer(self, os_, rank, capacity=None):
        """O_seq of one rank: [rows, H], column block d holds os_[d][rank*M:(rank+1)*M] flattened
        (tests/test_row_blocks.py:150-156)."""
        p = self.p
        m = os_[0].shape[0] // p
        rows = m if capacity is None else capacity
        out = torch.zeros(rows, self.h, dtype=os_[0].dtype)
        for dsrc in range(p):
            out[:m, dsrc * self.c:(dsrc + 1) * self.c] = os_[dsrc][rank * m:(rank + 1) * m].reshape(m, self.c)
        return out

    def out_forward(self, os_):
        """os_: list of P [P*M, N/P, D]. Returns list of P [M, H]. The bias is added in the
        activation dtype after rounding (fused_gemm_a2a.py:373-375)."""
        ys = []
        for r in range(self.p):
            y = _mm(self.out_recv_buffer(os_, r), self.wo.t(), self.acc).to(self.dtype)
            if self.bo is not None and self.apply_bias:
                y = (y.to(self.acc) + self.bo.to(self.acc)).to(self.dtype)
            ys.append(y)
        return ys

    def out_backward(self, os_, dys):
        """Returns (dOs: list of P [P*M, N/P, D] in dtype, per rank (dW [H,H], dbias [H]))."""
        p, hpr, d = self.p, self.n // self.p, self.d
        m = dys[0].shape[0]
        dos = [torch.zeros(p * m, hpr, d, dtype=self.dtype) for _ in range(p)]
        params = []
        for r, dy in enumerate(dys):
            full = _mm(dy, self.wo, self.acc).to(self.dtype)
            for dest in range(p):
                dos[dest][r * m:(r + 1) * m] = full[:, dest * self.c:(dest + 1) * self.c].reshape(m, hpr, d)
            params.append((_mm(dy.t(), self.out_recv_buffer(os_, r), self.acc), dy.to(self.acc).sum(0)))
        return dos, params

    def out_dhead_buffers(self, dys, capacity):
        """Head-side 'dhead' buffers after the output-projection dgrad push: per destination one
        [P*capacity, H/P] matrix, pad rows zero."""
        p = self.p
        bufs = [torch.zeros(p * capacity, self.c, dtype=self.dtype) for _ in range(p)]
        for r, dy in enumerate(dys):
            full = _mm(dy, self.wo, self.acc).to(self.dtype)
            for dest in range(p):
                bufs[dest][r * capacity:r * capacity + dy.shape[0]] = full[:, dest * self.c:(dest + 1) * self.c]
        return bufs


# ---------------------------------------------------------------------- auxiliary kernels
def resize_rank_rows_ref(tensors, peers, rows, *, bias=None, head_dim=128, head_offset=0):
    """out[r*rows + i] = in[r*in_rows + i] for i < min(rows, in_rows), zero otherwise; optional
    interleaved bias added in FP32 and rounded once, never on added rows
    (fused_gemm_a2a_kernels.py:1106-1142)."""
    outs = []
    segments = len(tensors)
    for s, t in enumerate(tensors):
        in_rows, width = t.shape[0] // peers, t.shape[1]
        out = torch.zeros(peers, rows, width, dtype=t.dtype)
        keep = min(rows, in_rows)
        vals = t.reshape(peers, in_rows, width)[:, :keep]
        if bias is not None:
            cols = torch.arange(width)
            idx = ((head_offset + cols // head_dim) * segments + s) * head_dim + cols % head_dim
            vals = (vals.float() + bias[idx].float()).to(t.dtype)
        out[:, :keep] = vals
        outs.append(out.reshape(peers * rows, width))
    return tuple(outs)


def reduce_bias_grad_ref(dy, out_dtype, previous=None):
    """Column sums in FP64 (the exact value an FP32 tree sum approximates), plus `previous` when
    accumulating, rounded once (fused_gemm_a2a_kernels.py:1086-1103)."""
    total = dy.double().sum(0)
    if previous is not None:
        total = total + previous.double()
    return total.to(out_dtype)


# ---------------------------------------------------------------------- grouped-query attention
def interleave_gqa_rows(segment_major, heads, kv_heads, head_dim, gate=False):
    """Rows in segment-major order [Q (heads); K (kv_heads); V (kv_heads)(; G (heads))] -> grouped
    order, one group per key/value head: [q_g0 .. q_g(r-1); k_g; v_g(; gate_g0 .. gate_g(r-1))]
    with r = heads / kv_heads. For r = 1 this is interleave_qkv_rows. The reference's unfused
    baseline keeps one weight per projection (benchmark/reference.py:151-163, with
    num_kv_heads < num_heads); the grouped order is Megatron's layout of a fused QKV weight under
    grouped-query attention."""
    r = heads // kv_heads
    if heads % kv_heads or segment_major.shape[0] != (heads * (2 if gate else 1) + 2 * kv_heads) * head_dim:
        raise ValueError('rows are not Q, K, V (and gate) blocks of these head counts')
    tail = tuple(segment_major.shape[1:])
    q_rows, kv_rows = heads * head_dim, kv_heads * head_dim
    q = segment_major[:q_rows].reshape((kv_heads, r, head_dim) + tail)
    k = segment_major[q_rows:q_rows + kv_rows].reshape((kv_heads, 1, head_dim) + tail)
    v = segment_major[q_rows + kv_rows:q_rows + 2 * kv_rows].reshape((kv_heads, 1, head_dim) + tail)
    parts = [q, k, v]
    if gate:
        parts.append(segment_major[q_rows + 2 * kv_rows:].reshape((kv_heads, r, head_dim) + tail))
    return torch.cat(parts, dim=1).reshape((-1,) + tail)


def deinterleave_gqa_rows(grouped, heads, kv_heads, head_dim, gate=False):
    """Inverse of interleave_gqa_rows."""
    r = heads // kv_heads
    per_group = r * (2 if gate else 1) + 2
    tail = tuple(grouped.shape[1:])
    g = grouped.reshape((kv_heads, per_group, head_dim) + tail)
    parts = [g[:, :r], g[:, r:r + 1], g[:, r + 1:r + 2]] + ([g[:, r + 2:]] if gate else [])
    return torch.cat([part.reshape((-1,) + tail) for part in parts], dim=0)


class GroupedQueryOracle(UlyssesOracle):
    """UlyssesOracle with fewer key/value heads than query heads. weight_qkv / bias_qkv are in the
    grouped row order of interleave_gqa_rows; outputs are q [P*M, N/P, D], k and v
    [P*M, Nkv/P, D] (and gate like q). The output projection is unchanged."""

    def __init__(self, p, hidden, heads, kv_heads, gate=False, **kwargs):
        if heads % kv_heads or kv_heads % p:
            raise ValueError('query heads must be a multiple of key/value heads, which must split over P')
        super().__init__(p, hidden, heads, 4 if gate else 3, **kwargs)
        self.kv, self.r, self.gate = kv_heads, heads // kv_heads, gate
        self.per_group = self.r * (2 if gate else 1) + 2
        # units of each kind inside a group: (first, count)
        self.kinds = [(0, self.r), (self.r, 1), (self.r + 1, 1)] + ([(self.r + 2, self.r)] if gate else [])

    def _by_kind(self, y):
        """[rows, Nkv*per_group*D] in weight-row order -> per kind [rows, heads of that kind, D]."""
        rows = y.shape[0]
        g = y.reshape(rows, self.kv, self.per_group, self.d)
        return [g[:, :, first:first + count].reshape(rows, self.kv * count, self.d) for first, count in self.kinds]

    def qkv_forward(self, xs):
        gpr = self.kv // self.p
        ys = [self._by_kind(self.qkv_sequence_side(x)) for x in xs]
        bias = None
        if self.bq is not None and self.apply_bias and not self.bias_in_gemm:
            bias = self._by_kind(self.bq.reshape(1, -1))
        outs = []
        for dest in range(self.p):
            per_kind = []
            for kind, (_, count) in enumerate(self.kinds):
                heads_of_dest = slice(dest * gpr * count, (dest + 1) * gpr * count)
                t = torch.cat([y[kind][:, heads_of_dest] for y in ys], dim=0).contiguous()
                if bias is not None:
                    t = (t.to(self.acc) + bias[kind][:, heads_of_dest].to(self.acc)).to(self.dtype)
                per_kind.append(t)
            outs.append(tuple(per_kind))
        return outs

    def qkv_heads_buffers(self, xs, capacity):
        gpr = self.kv // self.p
        bufs = [[torch.zeros(self.p * capacity, gpr * count * self.d, dtype=self.dtype) for _, count in self.kinds]
                for _ in range(self.p)]
        for r, x in enumerate(xs):
            xp = torch.zeros(capacity, self.h, dtype=x.dtype)
            xp[:x.shape[0]] = x
            y = self._by_kind(self.qkv_sequence_side(xp))
            for dest in range(self.p):
                for kind, (_, count) in enumerate(self.kinds):
                    bufs[dest][kind][r * capacity:(r + 1) * capacity] = \
                        y[kind][:, dest * gpr * count:(dest + 1) * gpr * count].reshape(capacity, -1)
        return bufs

    def qkv_recv_buffer(self, grads, rank, capacity=None):
        """dY of one rank in weight-row column order: grads[dest][kind] is [P*M, heads of that kind
        per rank, D]; group g of destination dest is global group dest*gpr + g."""
        gpr = self.kv // self.p
        m = grads[0][0].shape[0] // self.p
        rows = m if capacity is None else capacity
        out = torch.zeros(rows, self.kv, self.per_group, self.d, dtype=grads[0][0].dtype)
        for dest in range(self.p):
            for kind, (first, count) in enumerate(self.kinds):
                mine = grads[dest][kind][rank * m:(rank + 1) * m].reshape(m, gpr, count, self.d)
                out[:m, dest * gpr:(dest + 1) * gpr, first:first + count] = mine
        return out.reshape(rows, self.kv * self.per_group * self.d)
