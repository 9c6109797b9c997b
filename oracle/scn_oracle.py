"""CPU restatement of the INS-Conv sparse-convolution hot path.  TEST INFRASTRUCTURE ONLY.

Only tests/, __graft_entry__.smoke() and the cpu_baseline / reference legs of bench.py may import
this module, and only as the checker or the timed CPU baseline.  Nothing the library ships calls it.

PARITY PINNED AGAINST THE REFERENCE ITSELF: the reference repository holds no tests, golden vectors or
fixtures for this path, so the restatement is checked against the reference's own code run on the host:
oracle/build_ref.py compiles the reference's Metadata, rulebook builders and cuda_* / cpu_* operators from the
sources where they lie (its CUDA kernels run through a CUDA-on-host emulation; CUDPP, which its build vendors, is
stood in for by its documented contract -- unique-key rank, stable value order, scan, compact), and
tests/test_oracle_vs_reference.py compares every function of this module with it: site numbering, input rules,
3x3x3 and 2/2 rulebooks, every full-frame and incremental operator.  Outputs of the reference on seeded inputs are
committed as tests/golden/ref_*.npz (made by tests/golden/make_golden_ref.py) for machines without the reference
tree.  What the reference has no semantics for -- voxel deletion, an incremental mode that equals a full
recompute -- stays unpinned: it is checked against the full recompute only.
Each function cites the reference lines it follows (paths relative to sparseconvnet/SCN/ of
THU-luvision/INS-Conv).

Integer work (keys, site numbering, rulebooks) is numpy; floating point follows the reference's CPU
ops -- per offset index_select -> mm -> index_add_ on torch CPU tensors (CPU/Convolution.cpp:36-72).
"""
import numpy as np
import torch

MAX_COORD = 65534


# --------------------------------------------------------------------------------------------------
# keys and site numbering
# --------------------------------------------------------------------------------------------------
def ref_key31(x, y, z):
    """The reference's packed key, (z<<21 | y<<10 | x) & 0x7FFFFFFF (CUDA/CUDPPWrapper.cu:110-119).
    Valid (alias-free) only for x,z in [0,1023], y in [0,2047]."""
    x = np.asarray(x, dtype=np.int64)
    y = np.asarray(y, dtype=np.int64)
    z = np.asarray(z, dtype=np.int64)
    return ((z << 21) | (y << 10) | x) & 0x7FFFFFFF


def key64(x, y, z, b):
    """Wide key of the B200 build: batch<<48 | z<<32 | y<<16 | x.  For coordinates inside the reference's
    alias-free range it orders sites exactly as ref_key31 does inside each batch item, and batch items
    follow each other as the reference's per-batch grids do (row offset `ctr`,
    CUDA/SubmanifoldRules_cuda.cu:91-114)."""
    x = np.asarray(x, dtype=np.uint64)
    y = np.asarray(y, dtype=np.uint64)
    z = np.asarray(z, dtype=np.uint64)
    b = np.asarray(b, dtype=np.uint64)
    return (b << np.uint64(48)) | (z << np.uint64(32)) | (y << np.uint64(16)) | x


class Grid(object):
    """Active sites of one scale.

    keys   uint64 [n] ascending; row i <-> i-th smallest key (the CUDPP multivalue table gives every
           unique key the index of its rank: extra/cudpp/src/cudpp_hash/hash_multivalue.cpp:45-110)
    coords int64 [n,4] (x,y,z,batch) of each site (CUDA/CUDPPWrapper.cu:212-231)
    src_row int32 [n_src] source row (input point or finer site) -> site row (_d_hash_idx)
    """

    def __init__(self, coords_xyzb):
        c = np.asarray(coords_xyzb, dtype=np.int64)
        if c.ndim != 2 or c.shape[1] not in (3, 4):
            raise ValueError("coords must be [n,3] or [n,4]")
        if c.shape[1] == 3:
            c = np.concatenate([c, np.zeros((c.shape[0], 1), np.int64)], 1)
        if c.size and (c.min() < 0 or c[:, :3].max() > MAX_COORD):
            raise ValueError("coordinate outside the key range")
        k = key64(c[:, 0], c[:, 1], c[:, 2], c[:, 3])
        self.keys, first, inv = np.unique(k, return_index=True, return_inverse=True)
        self.n = int(self.keys.shape[0])
        self.n_src = int(c.shape[0])
        self.coords = c[first]
        self.src_row = inv.astype(np.int32).reshape(-1)

    def lookup(self, coords_xyzb):
        """Row of each coordinate or -1 (Multival_Point_Hashtable::retrieve, CUDA/CUDPPWrapper.hpp:900-1010).
        Coordinates outside the key range miss (the reference aliases them instead; parity tests stay
        inside its alias-free range)."""
        c = np.asarray(coords_xyzb, dtype=np.int64)
        ok = (c[:, :3] >= 0).all(1) & (c[:, :3] <= MAX_COORD).all(1) & (c[:, 3] >= 0)
        cc = np.where(ok[:, None], c, 0)
        k = key64(cc[:, 0], cc[:, 1], cc[:, 2], cc[:, 3])
        pos = np.searchsorted(self.keys, k)
        pos_c = np.minimum(pos, max(self.n - 1, 0))
        hit = ok & (self.n > 0)
        if self.n:
            hit &= self.keys[pos_c] == k
        return np.where(hit, pos_c, -1).astype(np.int32)

    def hash_contents(self):
        """The key -> row map a table must hold."""
        return dict(zip(self.keys.tolist(), range(self.n)))


# --------------------------------------------------------------------------------------------------
# InputLayer / OutputLayer
# --------------------------------------------------------------------------------------------------
def input_rules(grid, mode):
    """Reference layout (CUDA/IOLayers.cu:7-12, CUDA/CUDPPWrapper.cu:53-64): header
    [mode, maxActive, nIn, nOut]; rows [nOut, 1+maxActive] = count, then the point indices of the site
    in ascending order (stable radix sort of (key, index)), zero padded."""
    order = np.argsort(grid.src_row, kind="stable")
    counts = np.bincount(grid.src_row, minlength=grid.n).astype(np.int32)
    max_active = int(counts.max()) if grid.n else 0
    rows = np.zeros((grid.n, 1 + max_active), dtype=np.int32)
    rows[:, 0] = counts
    start = np.concatenate([[0], np.cumsum(counts)[:-1]]) if grid.n else np.zeros(0, np.int64)
    sorted_rows = grid.src_row[order]
    within = np.arange(grid.n_src) - start[sorted_rows]
    rows[sorted_rows, 1 + within] = order.astype(np.int32)
    header = np.array([mode, max_active, grid.n_src, grid.n], dtype=np.int32)
    return header, rows


def input_forward(feats, grid, mode):
    """InputLayer_ForwardPass (CPU/IOLayers.cpp:12-29): out[site] += multiplier * in[point] in rule order."""
    feats = torch.as_tensor(feats, dtype=torch.float32)
    _, rows = input_rules(grid, mode)
    out = torch.zeros(grid.n, feats.shape[1], dtype=torch.float32)
    cnt = torch.from_numpy(rows[:, 0].astype(np.int64))
    mult = torch.where(cnt > 0, 1.0 / cnt.clamp(min=1).float(), torch.ones(())) if mode == 4 else torch.ones(grid.n)
    for j in range(rows.shape[1] - 1):
        sel = torch.from_numpy(np.nonzero(rows[:, 0] > j)[0])
        if sel.numel() == 0:
            break
        idx = torch.from_numpy(rows[sel.numpy(), 1 + j].astype(np.int64))
        out[sel] += mult[sel, None] * feats[idx]
    return out


def output_forward(vox, grid):
    """OutputLayer (CUDA/IOLayers.cpp:123-145 -> InputLayer_bp_ with average=false): each point receives
    its site's row."""
    vox = torch.as_tensor(vox, dtype=torch.float32)
    return vox[torch.from_numpy(grid.src_row.astype(np.int64))]


# --------------------------------------------------------------------------------------------------
# rulebooks
# --------------------------------------------------------------------------------------------------
def ssc_offsets():
    """Offset order of the 3x3x3 filter: k = (dx+1)*9 + (dy+1)*3 + (dz+1), x slowest
    (CUDA/SubmanifoldRules_cuda.cu:61-74); the input site is output + (dx,dy,dz)."""
    return [(dx, dy, dz) for dx in (-1, 0, 1) for dy in (-1, 0, 1) for dz in (-1, 0, 1)]


def ssc_rules(grid, lookup_grid=None, only_rows=None):
    """27 arrays [R_k,2] of (input_row, output_row), ascending in output_row
    (_dGenerateRulebook + compaction, CUDA/SubmanifoldRules_cuda.cu:91-114).  lookup_grid / only_rows give
    the incremental variant: neighbours are looked up in the saved grid, only for the listed rows
    (IncreSubmanifoldBuildObject, CUDA/SubmanifoldRules_cuda.cpp:254-294)."""
    lg = grid if lookup_grid is None else lookup_grid
    rows = np.arange(grid.n, dtype=np.int32) if only_rows is None else np.asarray(only_rows, dtype=np.int32)
    rules = []
    for dx, dy, dz in ssc_offsets():
        q = grid.coords[rows].copy()
        q[:, 0] += dx
        q[:, 1] += dy
        q[:, 2] += dz
        r = lg.lookup(q)
        hit = r >= 0
        rules.append(np.stack([r[hit], rows[hit]], 1).astype(np.int32))
    return rules


def conv2_rules(fine):
    """Size-2 / stride-2 convolution (Convolution_InputSgToRulesAndOutputSg_FastDownSampleMode,
    Metadata/ConvolutionRules.h:344-380; _d_Convolution_GenerateOutputRules,
    CUDA/SubmanifoldRules_cuda.cu:744-780): coarse site = coord/2, numbered by key rank; offset
    k = (x&1)*4 + (y&1)*2 + (z&1); 8 arrays [R_k,2] of (fine_row, coarse_row), ascending in fine_row."""
    cc = fine.coords.copy()
    cc[:, :3] //= 2
    coarse = Grid(cc)
    k = (fine.coords[:, 0] & 1) * 4 + (fine.coords[:, 1] & 1) * 2 + (fine.coords[:, 2] & 1)
    rules = []
    for o in range(8):
        f = np.nonzero(k == o)[0].astype(np.int32)
        rules.append(np.stack([f, coarse.src_row[f]], 1).astype(np.int32))
    return coarse, rules


def canonical(rules):
    """Comparison form of a rulebook: per offset the pairs sorted by (output, input)."""
    out = []
    for r in rules:
        r = np.asarray(r, dtype=np.int32).reshape(-1, 2)
        out.append(r[np.lexsort((r[:, 0], r[:, 1]))])
    return out


# --------------------------------------------------------------------------------------------------
# feature math
# --------------------------------------------------------------------------------------------------
def conv_forward(x, weight, rules, n_out_rows, bias=None, reverse=False, out=None):
    """cpu_Convolution_updateOutput (CPU/Convolution.cpp:36-72): output = bias (or 0); per offset
    rows = index_select(input, rule[:,0]); output.index_add_(rule[:,1], mm(rows, W[k])).
    reverse=True swaps the pair, which is cpu_Deconvolution_updateOutput (CPU/Deconvolution.cpp:8-44)."""
    x = torch.as_tensor(x, dtype=torch.float32)
    weight = torch.as_tensor(weight, dtype=torch.float32)
    if out is None:
        out = torch.zeros(n_out_rows, weight.shape[2], dtype=torch.float32)
        if bias is not None and n_out_rows:
            out += torch.as_tensor(bias, dtype=torch.float32)
    for k, r in enumerate(rules):
        if len(r) == 0:
            continue
        r = torch.from_numpy(np.ascontiguousarray(r).astype(np.int64))
        i, o = (r[:, 1], r[:, 0]) if reverse else (r[:, 0], r[:, 1])
        out.index_add_(0, o, torch.mm(x.index_select(0, i), weight[k]))
    return out


def rule_flops(rules, n_in, n_out):
    return float(sum(len(r) for r in rules)) * n_in * n_out


def bn_forward(x, running_mean, running_var, gamma, beta, eps, leakiness):
    """BatchNormalization_ForwardPass, test mode (CPU/BatchNormalization.cpp:41-61)."""
    x = torch.as_tensor(x, dtype=torch.float32)
    w = torch.pow(torch.as_tensor(running_var, dtype=torch.float32) + eps, -0.5)
    if gamma is not None:
        w = w * torch.as_tensor(gamma, dtype=torch.float32)
    b = -torch.as_tensor(running_mean, dtype=torch.float32) * w
    if beta is not None:
        b = b + torch.as_tensor(beta, dtype=torch.float32)
    o = x * w + b
    return torch.where(o > 0, o, o * leakiness)


def bn_forward_train(x, running_mean, running_var, gamma, beta, eps, momentum, leakiness):
    """BatchNormalization_ForwardPass, train mode (CPU/BatchNormalization.cpp:22-40): batch statistics, running
    statistics updated as momentum*running + (1-momentum)*batch with the unbiased variance.  Returns
    (out, new_running_mean, new_running_var)."""
    x = torch.as_tensor(x, dtype=torch.float32)
    n = x.shape[0]
    xd = x.double()
    mean = xd.mean(0)
    ss = (xd * xd).sum(0) - mean * mean * n
    new_rm = momentum * torch.as_tensor(running_mean, dtype=torch.float32) + (1 - momentum) * mean.float()
    new_rv = momentum * torch.as_tensor(running_var, dtype=torch.float32) + (1 - momentum) * (ss / (n - 1)).float()
    out = bn_forward(x, mean.float(), (ss / n).float(), gamma, beta, eps, leakiness)
    return out, new_rm, new_rv


def nin_forward(x, weight, bias=None):
    """cpu_NetworkInNetwork_updateOutput (CPU/NetworkInNetwork.cpp:8-23)."""
    x = torch.as_tensor(x, dtype=torch.float32)
    out = torch.mm(x, torch.as_tensor(weight, dtype=torch.float32))
    if bias is not None:
        out = out + torch.as_tensor(bias, dtype=torch.float32)
    return out


# --------------------------------------------------------------------------------------------------
# incremental path (reference semantics: insert-only, no dilation of the changed set)
# --------------------------------------------------------------------------------------------------
def pre_exist(grid, pre_grid):
    """Metadata::getPreExistMaps (Metadata/Metadata.cpp:609-626): row in the saved grid or -1."""
    return pre_grid.lookup(grid.coords)


def incre_input_forward(feats, grid, mode, pre_grid, pre_out):
    """InputLayer_inc_fp_ (CUDA/IOLayers.cu:82-106): mult = 1/(n_new + n_saved) for mode 4;
    out = sum(mult * new) + saved * (n_saved * mult - 1)."""
    feats = torch.as_tensor(feats, dtype=torch.float32)
    pre_out = torch.as_tensor(pre_out, dtype=torch.float32)
    _, rows = input_rules(grid, mode)
    pe = pre_exist(grid, pre_grid)
    pre_cnt_all = np.bincount(pre_grid.src_row, minlength=pre_grid.n)
    pre_cnt = np.where(pe >= 0, pre_cnt_all[np.maximum(pe, 0)], 0)
    cnt = rows[:, 0].astype(np.int64)
    if mode == 4:
        mult = np.where(cnt > 0, 1.0 / np.maximum(cnt + pre_cnt, 1).astype(np.float32), 1.0).astype(np.float32)
    else:
        mult = np.ones(grid.n, np.float32)
    mult_t = torch.from_numpy(mult)
    out = torch.zeros(grid.n, feats.shape[1], dtype=torch.float32)
    for j in range(rows.shape[1] - 1):
        sel = np.nonzero(rows[:, 0] > j)[0]
        if sel.size == 0:
            break
        idx = torch.from_numpy(rows[sel, 1 + j].astype(np.int64))
        selt = torch.from_numpy(sel)
        out[selt] += mult_t[selt, None] * feats[idx]
    ex = np.nonzero(pe >= 0)[0]
    if ex.size:
        ext = torch.from_numpy(ex)
        f = torch.from_numpy((pre_cnt[ex].astype(np.float32) * mult[ex] - np.float32(1.0)).astype(np.float32))
        out[ext] = out[ext] + pre_out[torch.from_numpy(pe[ex].astype(np.int64))] * f[:, None]
    return out


def incre_output_forward(vox, grid, pre_grid, pre_in):
    """InputLayer_inc_bp_ (CUDA/IOLayers.cu:123-142): point = residual row + saved row when the site existed."""
    vox = torch.as_tensor(vox, dtype=torch.float32)
    pre_in = torch.as_tensor(pre_in, dtype=torch.float32)
    pe = pre_exist(grid, pre_grid)
    full = vox.clone()
    ex = np.nonzero(pe >= 0)[0]
    if ex.size:
        full[torch.from_numpy(ex)] += pre_in[torch.from_numpy(pe[ex].astype(np.int64))]
    return full[torch.from_numpy(grid.src_row.astype(np.int64))]


def incre_ssc_rules(grid, pre_grid):
    """Rules (pre_row_of_neighbour, row) for the sites of `grid` that are absent from the saved grid."""
    pe = pre_exist(grid, pre_grid)
    return ssc_rules(grid, lookup_grid=pre_grid, only_rows=np.nonzero(pe < 0)[0])


def incre_ssc_forward(x_res, weight, grid, pre_grid, pre_x, bias=None):
    """cuda_Incre_SubmanifoldConvolution_updateOutput (CUDA/Convolution.cpp:221-303)."""
    out = conv_forward(x_res, weight, ssc_rules(grid), grid.n, bias)
    return conv_forward(pre_x, weight, incre_ssc_rules(grid, pre_grid), grid.n, out=out)


def incre_bn_forward(x_res, running_mean, running_var, gamma, beta, eps, leakiness, grid, pre_grid, pre_out, pre_in):
    """Incre_BatchNormalization_f_test (CUDA/BatchNormalization.cu:112-150)."""
    x_res = torch.as_tensor(x_res, dtype=torch.float32)
    pre_out = torch.as_tensor(pre_out, dtype=torch.float32)
    pre_in = torch.as_tensor(pre_in, dtype=torch.float32)
    w = torch.pow(torch.as_tensor(running_var, dtype=torch.float32) + eps, -0.5)
    if gamma is not None:
        w = w * torch.as_tensor(gamma, dtype=torch.float32)
    b = -torch.as_tensor(running_mean, dtype=torch.float32) * w
    if beta is not None:
        b = b + torch.as_tensor(beta, dtype=torch.float32)
    o = x_res * w + b
    y = torch.where(o > 0, o, o * leakiness)
    pe = pre_exist(grid, pre_grid)
    ex = np.nonzero(pe >= 0)[0]
    if ex.size:
        ext = torch.from_numpy(ex)
        pr = torch.from_numpy(pe[ex].astype(np.int64))
        v = o[ext] + pre_in[pr] * w
        y[ext] = torch.where(v > 0, v, v * leakiness) - pre_out[pr]
    return y


def incre_deconv_forward(x_res, weight, fine, coarse, rules, pre_fine, pre_coarse, pre_x, bias=None):
    """cuda_Incre_Deconvolution_updateOutput (CUDA/Deconvolution.cpp:61-96, CUDA/Deconvolution.cu:118-135):
    input row = residual row (+ saved row when the coarse site existed and the fine site is new)."""
    out = conv_forward(x_res, weight, rules, fine.n, bias, reverse=True)
    pe_c = pre_exist(coarse, pre_coarse)
    pe_f = pre_exist(fine, pre_fine)
    extra = []
    for r in rules:
        r = np.asarray(r).reshape(-1, 2)
        keep = (pe_c[r[:, 1]] >= 0) & (pe_f[r[:, 0]] < 0)
        extra.append(np.stack([r[keep, 0], pe_c[r[keep, 1]]], 1).astype(np.int32))
    return conv_forward(pre_x, weight, extra, fine.n, reverse=True, out=out)
