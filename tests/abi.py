"""ctypes binding of the C ABI (include/gsb200.h) for the tests: device memory comes from
torch, everything else goes through the shared library exactly as a foreign host would."""
import ctypes as C
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "gsb200.h")
LIB = os.path.join(ROOT, "gsampler_b200", "libgsb200.so")

I32, I64 = 0, 1


def declared_symbols():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"GSB_API\s+[\w\s\*]+?\b(gsb_\w+)\s*\(", text)))


_lib = None


def lib():
    global _lib
    if _lib is None:
        _lib = C.CDLL(LIB)
        for name in declared_symbols():
            fn = getattr(_lib, name)
            if name.endswith("_workspace_bytes"):
                fn.restype = C.c_size_t
            elif name in ("gsb_status_string", "gsb_last_cuda_error"):
                fn.restype = C.c_char_p
            else:
                fn.restype = C.c_int
    return _lib


def ptr(t):
    return C.c_void_p(0 if t is None else t.data_ptr())


def i64(v):
    return C.c_int64(int(v))


class LayerBuffers(C.Structure):
    _fields_ = [("S_cap", C.c_int64), ("E_cap", C.c_int64)] + [
        (n, C.c_void_p) for n in ("sub_indptr", "rows", "cols", "sel", "edge_ptr", "unique",
                                  "unique_ptr", "block_row", "block_col")]


def check(rc, what):
    if rc != 0:
        raise RuntimeError("%s -> %s (%s)" % (what, lib().gsb_status_string(rc).decode(),
                                              lib().gsb_last_cuda_error().decode()))


# ------------------------------------------------------------------ thin call helpers
def sample_cols(indptr, indices, seeds, K, replace, seed, stream, S=None, d_S=None, E_cap=None,
                probs=None, num_cols=None):
    import torch

    dev = indptr.device
    ncols = indptr.numel() - 1 if num_cols is None else num_cols
    S_max = int(seeds.numel() if seeds is not None else indptr.numel() - 1) if S is None else S
    E_cap = S_max * K if E_cap is None else E_cap
    o = dict(dtype=torch.int64, device=dev)
    sub = torch.full((S_max + 1,), -7, **o)
    rows, cols, sel = (torch.full((E_cap,), -7, **o) for _ in range(3))
    scal = torch.zeros(2, **o)
    err = torch.zeros(1, dtype=torch.int32, device=dev)
    dt = I32 if indices.dtype == torch.int32 else I64
    L = lib()
    st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    if probs is None:
        nb = L.gsb_sample_cols_workspace_bytes(i64(S_max), i64(K))
        ws = torch.empty(nb + 256, dtype=torch.uint8, device=dev)
        rc = L.gsb_sample_cols(ptr(indptr), ptr(indices), dt, i64(ncols), ptr(seeds), i64(S_max), ptr(d_S),
                               i64(K), int(replace), C.c_uint64(seed), C.c_uint32(stream), ptr(sub),
                               ptr(rows), ptr(cols), ptr(sel), i64(E_cap), ptr(scal), ptr(ws),
                               C.c_size_t(ws.numel()), ptr(err), st)
    else:
        nb = L.gsb_sample_cols_probs_workspace_bytes(i64(S_max), i64(K))
        ws = torch.empty(nb + 256, dtype=torch.uint8, device=dev)
        rc = L.gsb_sample_cols_probs(ptr(indptr), ptr(indices), dt, i64(ncols), ptr(probs), ptr(seeds),
                                     i64(S_max), ptr(d_S), i64(K), int(replace), C.c_uint64(seed),
                                     C.c_uint32(stream), ptr(sub), ptr(rows), ptr(cols), ptr(sel),
                                     i64(E_cap), ptr(scal), ptr(ws), C.c_size_t(ws.numel()),
                                     ptr(err), st)
    check(rc, "gsb_sample_cols")
    torch.cuda.synchronize()
    E = int(scal[0])
    return sub, rows[:E], cols[:E], sel[:E], int(err[0])


def slice_cols(indptr, indices, seeds, col_bptr=None, encoding_size=0):
    import torch

    dev = indptr.device
    S = seeds.numel()
    o = dict(dtype=torch.int64, device=dev)
    sub = torch.empty(S + 1, **o)
    err = torch.zeros(1, dtype=torch.int32, device=dev)
    L = lib()
    st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    ws = torch.empty(L.gsb_slice_cols_workspace_bytes(i64(S)) + 256, dtype=torch.uint8, device=dev)
    check(L.gsb_slice_cols_count(ptr(indptr), i64(indptr.numel() - 1), ptr(seeds), i64(S), ptr(sub), ptr(ws),
                                 C.c_size_t(ws.numel()), ptr(err), st), "gsb_slice_cols_count")
    E = int(sub[S])
    rows, cols, sel = (torch.empty(E, **o) for _ in range(3))
    dt = I32 if indices.dtype == torch.int32 else I64
    B = 0 if col_bptr is None else col_bptr.numel() - 1
    check(L.gsb_slice_cols_fill(ptr(indptr), ptr(indices), dt, ptr(seeds), i64(S), ptr(sub), i64(E),
                                ptr(rows), ptr(cols), ptr(sel), ptr(col_bptr), i64(B),
                                i64(encoding_size), st), "gsb_slice_cols_fill")
    torch.cuda.synchronize()
    return sub, rows, cols, sel, int(err[0])


def batch_relabel(seeds, seeds_ptr, coo_row, coo_col, edge_ptr, want_edges=True, U_cap=None,
                  id_bound=0):
    import torch

    dev = seeds_ptr.device
    S, E, B = seeds.numel(), coo_row.numel(), seeds_ptr.numel() - 1
    o = dict(dtype=torch.int64, device=dev)
    U_cap = S + E if U_cap is None else U_cap
    unique = torch.full((U_cap,), -7, **o)
    uptr = torch.full((B + 1,), -7, **o)
    orow = torch.full((E,), -7, **o) if want_edges else None
    ocol = torch.full((E,), -7, **o) if want_edges else None
    err = torch.zeros(1, dtype=torch.int32, device=dev)
    L = lib()
    st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    ws = torch.empty(L.gsb_batch_relabel_workspace_bytes(i64(S), i64(E), i64(B)) + 256,
                     dtype=torch.uint8, device=dev)
    check(L.gsb_batch_relabel(ptr(seeds), ptr(seeds_ptr), i64(B), i64(S), ptr(coo_row),
                              ptr(coo_col if want_edges else None), ptr(edge_ptr), i64(E), i64(id_bound),
                              ptr(unique), i64(U_cap), ptr(uptr), ptr(orow), ptr(ocol), ptr(ws),
                              C.c_size_t(ws.numel()), ptr(err), st), "gsb_batch_relabel")
    torch.cuda.synchronize()
    U = int(uptr[B])
    return unique[:max(U, 0)], uptr, orow, ocol, int(err[0])


def random_walk(indptr, indices, seeds, length, seed, stream, indptr32=None, node2vec=None):
    """gsb_random_walk / gsb_node2vec (``node2vec`` = (p, q)); returns (trace [(L+1) * N], error word)."""
    import torch

    N = seeds.numel()
    out = torch.empty(N * (length + 1), dtype=torch.int64, device="cuda")
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    dt = I32 if indices.dtype == torch.int32 else I64
    num_nodes = (indptr if indptr is not None else indptr32).numel() - 1
    st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    if node2vec is None:
        check(lib().gsb_random_walk(ptr(indptr), ptr(indptr32), ptr(indices), dt, i64(num_nodes), ptr(seeds),
                                    i64(N), i64(length), C.c_uint64(seed), C.c_uint32(stream), ptr(out),
                                    ptr(err), st), "gsb_random_walk")
    else:
        check(lib().gsb_node2vec(ptr(indptr), ptr(indptr32), ptr(indices), dt, i64(num_nodes), ptr(seeds),
                                 i64(N), i64(length), C.c_double(node2vec[0]), C.c_double(node2vec[1]),
                                 C.c_uint64(seed), C.c_uint32(stream), ptr(out), ptr(err), st), "gsb_node2vec")
    return out, int(err.item())


def list_sample_whole(n, K, seed, stream):
    """gsb_list_sample on ONE list [0, n) stated by the caller: no offsets in, none out, no workspace."""
    import torch

    out = torch.empty(min(n, K), dtype=torch.int64, device="cuda")
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    check(lib().gsb_list_sample(None, None, i64(1), i64(n), i64(K), C.c_uint64(seed), C.c_uint32(stream),
                                ptr(out), None, None, C.c_size_t(0), ptr(err),
                                C.c_void_p(torch.cuda.current_stream().cuda_stream)), "gsb_list_sample")
    return out, int(err.item())
