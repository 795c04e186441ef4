"""TurboQuantIndex -- brute-force inner-product search over TurboQuant-compressed vectors, B200 build.

Same surface as upstream ``turboquant_kv/search.py:37-317`` (constructor, ``from_vectors``, ``add``,
``search``, ``save``, ``load``).  The database lives in GPU memory in the upstream packed layout;
``add`` runs the fused quantise kernel, ``search`` (MSE mode) runs the streaming packed-code scan with
top-k selection (csrc/scan.cu), which replaces both the Python path (unpack everything, gather an
(N, d) float matrix, one (Q, N) matmul, torch.topk; search.py:206-227) and the optional C++ core
(csrc/core/turboquant_core.cpp:407-514).

Tensors may be passed on the host or on the GPU; results come back on the device of the queries.
Results: scores descending, ids int64; equal scores are ordered by ascending id; ``k`` is clipped
to the number of stored vectors like the upstream Python path.

Prod mode (upstream search.py:229-252 reconstructs every row and multiplies by the queries) runs the same
scan over the packed Algorithm-2 rows: <q, x~> = norm * (<R q, c[codes]> + sqrt(pi/2)/d * ||r|| * <S q, signs>),
``tqb_scan_topk_prod`` -- no dense reconstruction of the database.
"""
from __future__ import annotations

import ctypes
import struct
from typing import Optional, Tuple

import torch

from . import _native as N
from .reference import _make_qjl_matrix, lloyd_max_codebook, make_rotation_matrix, quantize_mse, quantize_prod

HEADER_FORMAT = "<BII"  # bit_width (u8), dim (u32), n_vectors (u32) -- upstream search.py:29
HEADER_SIZE = struct.calcsize(HEADER_FORMAT)
MODE_MSE, MODE_PROD = 0, 1
TQIX_MAGIC, TQIX_VERSION = 0x54514958, 1  # upstream csrc/core/turboquant_core.cpp:520-521

_QUERY_CHUNK = 1024     # queries per scan call (bounds the candidate workspace)


def merge_topk(scores: torch.Tensor, ids: torch.Tensor, k: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """Merge per-shard results.  scores / ids: (Q, parts, k); entries with id -1 are padding.

    Ordering rule of the scan: score descending, then id ascending.  CUDA tensors go through the
    merge kernel; host tensors (used by the multi-process logic on CPU ranks) through a stable sort.
    """
    q, parts, kk = scores.shape
    if scores.is_cuda and kk == k:
        s = scores.contiguous().float()
        i = ids.contiguous().to(torch.int64)
        out_s = torch.empty(q, k, dtype=torch.float32, device=s.device)
        out_i = torch.empty(q, k, dtype=torch.int64, device=s.device)
        with torch.cuda.device(s.device):
            N.check(N.lib().tqb_topk_merge(N.ptr(s), N.ptr(i), q, parts, k, N.ptr(out_s), N.ptr(out_i),
                                           N.stream_of(s)))
        return out_s, out_i
    s = scores.reshape(q, parts * kk).float()
    i = ids.reshape(q, parts * kk).to(torch.int64)
    s = torch.where(i < 0, torch.full_like(s, float("-inf")), s)
    big = torch.where(i < 0, torch.full_like(i, torch.iinfo(torch.int64).max), i)
    order = torch.argsort(big, dim=1, stable=True)                      # id ascending ...
    s1, i1 = torch.gather(s, 1, order), torch.gather(i, 1, order)
    order = torch.argsort(s1, dim=1, descending=True, stable=True)      # ... then score descending
    s2, i2 = torch.gather(s1, 1, order)[:, :k], torch.gather(i1, 1, order)[:, :k]
    if s2.shape[1] < k:
        pad = k - s2.shape[1]
        s2 = torch.cat([s2, s2.new_full((q, pad), float("-inf"))], 1)
        i2 = torch.cat([i2, i2.new_full((q, pad), -1)], 1)
    return s2, i2


class TurboQuantIndex:
    """Compressed vector index; ``mode`` "mse" (Algorithm 1) or "prod" (Algorithm 2)."""

    def __init__(self, dim: int, bit_width: int = 3, mode: str = "mse", rotation: str = "dense_qr",
                 seed: int = 42, device=None):
        if mode not in ("mse", "prod"):
            raise ValueError(f"Unknown mode: {mode}")
        N.require_cuda()
        self.dim, self.bit_width, self.mode = dim, bit_width, mode
        self.rotation_method, self.seed = rotation, seed
        self.device = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
        self._use_cpp = False  # upstream attribute: no host C++ core in this build
        self._rotation = make_rotation_matrix(dim, seed=seed, method=rotation).to(self.device)
        mse_bits = bit_width if mode == "mse" else bit_width - 1
        if mode == "prod" and mse_bits < 1:
            raise ValueError(f"Prod mode requires bits >= 2, got {bit_width}")
        self._codebook = tuple(t.to(self.device) for t in lloyd_max_codebook(mse_bits, dim))
        self._S_matrix = _make_qjl_matrix(dim, dim, seed, self.device) if mode == "prod" else None
        # MSE indexes of dim 64 / 128 with 2-4 bits live on the GPU as key-only 16-row records
        # (csrc/tiled_layout.cuh), the layout the scan kernel streams; _packed_codes / _norms are then
        # exported upstream-layout copies.  Every other index keeps upstream rows.
        self._use_records = mode == "mse" and dim in (64, 128) and 2 <= bit_width <= 4
        self._records: Optional[torch.Tensor] = None
        self._rec_bytes = int(N.lib().tqb_kv_record_bytes(dim, bit_width, 0)) if self._use_records else 0
        self._rows_pc: Optional[torch.Tensor] = None     # upstream rows (stored, or cached export)
        self._rows_nm: Optional[torch.Tensor] = None
        self._qjl_signs: Optional[torch.Tensor] = None
        self._residual_norms: Optional[torch.Tensor] = None
        self.n_vectors = 0
        self.id_offset = 0           # added to every returned id (row-sharded indexes)
        self._workspace: Optional[torch.Tensor] = None

    @classmethod
    def from_vectors(cls, vectors: torch.Tensor, bit_width: int = 3, mode: str = "mse",
                     rotation: str = "dense_qr", seed: int = 42, device=None) -> "TurboQuantIndex":
        idx = cls(dim=vectors.shape[-1], bit_width=bit_width, mode=mode, rotation=rotation, seed=seed, device=device)
        idx.add(vectors)
        return idx

    # ---- upstream attribute names (search.py:96-99) -------------------------------------------
    def _export_rows(self) -> None:
        if self._rows_pc is not None or not self._use_records or self.n_vectors == 0:
            return
        n, bpp = self.n_vectors, (self.dim + 7) // 8
        pc = torch.empty(n, self.bit_width * bpp, dtype=torch.uint8, device=self.device)
        nm = torch.empty(n, dtype=torch.float32, device=self.device)
        with torch.cuda.device(self.device):
            N.check(N.lib().tqb_kv_export(N.ptr(self._records), n, self.dim, self.bit_width, 0, None, N.ptr(pc),
                                          N.ptr(nm), None, None, N.stream_of(pc)))
        self._rows_pc, self._rows_nm = pc, nm

    @property
    def _packed_codes(self) -> Optional[torch.Tensor]:
        self._export_rows()
        return self._rows_pc

    @_packed_codes.setter
    def _packed_codes(self, value: Optional[torch.Tensor]) -> None:
        self._rows_pc = value

    @property
    def _norms(self) -> Optional[torch.Tensor]:
        self._export_rows()
        return self._rows_nm

    @_norms.setter
    def _norms(self, value: Optional[torch.Tensor]) -> None:
        self._rows_nm = value

    def _reserve_records(self, rows: int) -> None:
        have = 0 if self._records is None else self._records.numel() // self._rec_bytes * 16
        if rows <= have:
            return
        cap = max(4096, have)
        while cap < rows:
            cap *= 2
        new = torch.zeros((cap // 16) * self._rec_bytes, dtype=torch.uint8, device=self.device)
        if self._records is not None:
            new[: self._records.numel()] = self._records
        self._records = new

    def _import_rows(self, packed: torch.Tensor, norms: torch.Tensor) -> None:
        """Upstream rows -> records (used by load())."""
        n = packed.shape[0]
        self._reserve_records(n)
        pc, nm = packed.to(self.device).contiguous(), norms.to(self.device, torch.float32).contiguous()
        with torch.cuda.device(self.device):
            N.check(N.lib().tqb_kv_import(N.ptr(self._records), n, self.dim, self.bit_width, 0, None, N.ptr(pc),
                                          N.ptr(nm), None, None, N.stream_of(pc)))
        self._rows_pc = self._rows_nm = None

    # ------------------------------------------------------------------------------------------
    @staticmethod
    def _grow(old: Optional[torch.Tensor], new: torch.Tensor) -> torch.Tensor:
        return new if old is None else torch.cat([old, new], dim=0)

    def add(self, vectors: torch.Tensor):
        """Quantise and append (N, dim) or (dim,) vectors."""
        if vectors.dim() == 1:
            vectors = vectors.unsqueeze(0)
        assert vectors.shape[-1] == self.dim
        x = vectors.to(self.device)
        if self._use_records:
            if x.dtype not in (torch.float32, torch.float16, torch.bfloat16):
                x = x.float()
            x = x.contiguous()
            n = x.shape[0]
            self._reserve_records(self.n_vectors + n)
            rm = N.RowMap(1, 1, 0, self.n_vectors, None, 1, None, 1)      # row r -> slot n_vectors + r
            with torch.cuda.device(self.device):
                N.check(N.lib().tqb_kv_append(N.ptr(x), None, N.dtype_code(x.dtype), n, self.dim, self.dim,
                                              N.ptr(self._rotation), N.ptr(self._codebook[0]), self.bit_width,
                                              None, None, 0, N.ptr(self._records), ctypes.byref(rm),
                                              N.stream_of(x)))
            self._rows_pc = self._rows_nm = None
            self.n_vectors += n
            return
        if self.mode == "mse":
            packed, norms = quantize_mse(x, self.bit_width, dim=self.dim, rotation=self._rotation,
                                         codebook=self._codebook)
        else:
            packed, signs, res, norms = quantize_prod(x, self.bit_width, dim=self.dim, rotation=self._rotation,
                                                      codebook=self._codebook, S_matrix=self._S_matrix)
            self._qjl_signs = self._grow(self._qjl_signs, signs)
            self._residual_norms = self._grow(self._residual_norms, res)
        self._packed_codes = self._grow(self._packed_codes, packed)
        self._norms = self._grow(self._norms, norms)
        self.n_vectors += x.shape[0]

    # ------------------------------------------------------------------------------------------
    def search(self, queries: torch.Tensor, k: int = 10) -> Tuple[torch.Tensor, torch.Tensor]:
        """Top-k inner products: (scores (Q, k) float32, ids (Q, k) int64)."""
        if queries.dim() == 1:
            queries = queries.unsqueeze(0)
        assert self.n_vectors > 0, "Index is empty"
        home = queries.device
        q = queries.to(self.device, torch.float32).contiguous()
        k = min(k, self.n_vectors)
        scores, ids = (self._search_mse if self.mode == "mse" else self._search_prod)(q, k)
        return scores.to(home), ids.to(home)

    def _search_mse(self, q: torch.Tensor, k: int):
        if k > N.SCAN_MAX_K:
            raise RuntimeError(f"k = {k} exceeds the scan's limit of {N.SCAN_MAX_K}")
        nq = q.shape[0]
        out_s = torch.empty(nq, k, dtype=torch.float32, device=self.device)
        out_i = torch.empty(nq, k, dtype=torch.int64, device=self.device)
        L = N.lib()
        with torch.cuda.device(self.device):
            for lo in range(0, nq, _QUERY_CHUNK):
                qc = q[lo:lo + _QUERY_CHUNK]
                n = qc.shape[0]
                if self._use_records:
                    need = L.tqb_scan_records_workspace_bytes(n, self.dim, self.bit_width, k)
                    if self._workspace is None or self._workspace.numel() < need:
                        self._workspace = torch.empty(need, dtype=torch.uint8, device=self.device)
                    N.check(L.tqb_scan_records_topk(N.ptr(qc), n, N.ptr(self._records), self.n_vectors, self.dim,
                                                    self.bit_width, N.ptr(self._rotation), N.ptr(self._codebook[1]),
                                                    k, self.id_offset, N.ptr(self._workspace),
                                                    self._workspace.numel(), N.ptr(out_s[lo:lo + n]),
                                                    N.ptr(out_i[lo:lo + n]), N.stream_of(qc)))
                    continue
                need = L.tqb_scan_topk_workspace_bytes(n, self.n_vectors, self.dim, self.bit_width, k)
                if self._workspace is None or self._workspace.numel() < need:
                    self._workspace = torch.empty(need, dtype=torch.uint8, device=self.device)
                N.check(L.tqb_scan_topk(N.ptr(qc), n, N.ptr(self._packed_codes), N.ptr(self._norms),
                                        self.n_vectors, self.dim, self.bit_width, N.ptr(self._rotation),
                                        N.ptr(self._codebook[1]), k, self.id_offset, N.ptr(self._workspace),
                                        self._workspace.numel(), N.ptr(out_s[lo:lo + n]), N.ptr(out_i[lo:lo + n]),
                                        N.stream_of(qc)))
        return out_s, out_i

    def _search_prod(self, q: torch.Tensor, k: int):
        """Prod-mode search over the packed rows (upstream search.py:229-252 dequantises every row and multiplies
        by the queries): <q, x~> = norm * (<R q, c[codes]> + sqrt(pi/2)/d * ||r|| * <S q, signs>), streamed row by
        row by the scan kernel, top-k merged on the GPU -- no dense reconstruction of the database."""
        if k > N.SCAN_MAX_K:
            raise RuntimeError(f"k = {k} exceeds the scan's limit of {N.SCAN_MAX_K}")
        L = N.lib()
        nq = q.shape[0]
        out_s = torch.empty(nq, k, dtype=torch.float32, device=self.device)
        out_i = torch.empty(nq, k, dtype=torch.int64, device=self.device)
        with torch.cuda.device(self.device):
            for lo in range(0, nq, _QUERY_CHUNK):
                qc = q[lo:lo + _QUERY_CHUNK].contiguous()
                n = qc.shape[0]
                need = L.tqb_scan_topk_prod_workspace_bytes(n, self.n_vectors, self.dim, self.bit_width, k)
                if self._workspace is None or self._workspace.numel() < need:
                    self._workspace = torch.empty(need, dtype=torch.uint8, device=self.device)
                N.check(L.tqb_scan_topk_prod(N.ptr(qc), n, N.ptr(self._packed_codes), N.ptr(self._qjl_signs),
                                             N.ptr(self._residual_norms), N.ptr(self._norms), self.n_vectors, self.dim,
                                             self.bit_width, N.ptr(self._rotation), N.ptr(self._codebook[1]),
                                             N.ptr(self._S_matrix), k, self.id_offset, N.ptr(self._workspace),
                                             self._workspace.numel(), N.ptr(out_s[lo:lo + n]), N.ptr(out_i[lo:lo + n]),
                                             N.stream_of(qc)))
        return out_s, out_i

    # ------------------------------------------------------------------------------------------
    def save(self, path: str, format: str = "python"):
        """Write the index.  "python": upstream search.py:254-277 (header <BII, mode byte, codes, norms
        [, signs, residual norms]).  "tqix": upstream C++ core layout, MSE only
        (csrc/core/turboquant_core.cpp:559-580: magic, version, dim, bits, seed, n as u32, codes, norms)."""
        codes = self._packed_codes.cpu().numpy().tobytes() if self.n_vectors else b""
        norms = self._norms.cpu().numpy().tobytes() if self.n_vectors else b""
        with open(path, "wb") as f:
            if format == "tqix":
                if self.mode != "mse":
                    raise ValueError("the TQIX layout stores MSE indexes only")
                f.write(struct.pack("<6I", TQIX_MAGIC, TQIX_VERSION, self.dim, self.bit_width,
                                    self.seed & 0xFFFFFFFF, self.n_vectors))
                f.write(codes)
                f.write(norms)
                return
            if format != "python":
                raise ValueError(f"Unknown format: {format}")
            f.write(struct.pack(HEADER_FORMAT, self.bit_width, self.dim, self.n_vectors))
            f.write(struct.pack("<B", MODE_MSE if self.mode == "mse" else MODE_PROD))
            f.write(codes)
            f.write(norms)
            if self.mode == "prod" and self.n_vectors:
                f.write(self._qjl_signs.cpu().numpy().tobytes())
                f.write(self._residual_norms.cpu().numpy().tobytes())

    @classmethod
    def load(cls, path: str, rotation: str = "dense_qr", seed: int = 42, device=None) -> "TurboQuantIndex":
        """Read either on-disk layout (recognised by the TQIX magic)."""
        import numpy as np

        with open(path, "rb") as f:
            blob = f.read()
        if len(blob) >= 24 and struct.unpack_from("<I", blob, 0)[0] == TQIX_MAGIC:
            _, version, dim, bits, file_seed, n = struct.unpack_from("<6I", blob, 0)
            if version != TQIX_VERSION:
                raise RuntimeError("Unsupported TQIDX version")
            mode, off, seed = "mse", 24, file_seed
        else:
            bits, dim, n = struct.unpack_from(HEADER_FORMAT, blob, 0)
            mode = "mse" if blob[HEADER_SIZE] == MODE_MSE else "prod"
            off = HEADER_SIZE + 1
        bpp = (dim + 7) // 8
        pbytes = (bits if mode == "mse" else bits - 1) * bpp

        def take(count, dtype, width):
            nonlocal off
            nbytes = count * width
            if off + nbytes > len(blob):
                raise RuntimeError(f"Read error / truncated file: {path}")
            arr = np.frombuffer(blob, dtype=dtype, count=nbytes // np.dtype(dtype).itemsize, offset=off).copy()
            off += nbytes
            return torch.from_numpy(arr)

        idx = cls(dim=dim, bit_width=bits, mode=mode, rotation=rotation, seed=seed, device=device)
        packed = take(n, np.uint8, pbytes).reshape(n, pbytes)
        norms = take(n, np.float32, 4)
        if idx._use_records and n:
            idx._import_rows(packed, norms)
        else:
            idx._packed_codes = packed.to(idx.device)
            idx._norms = norms.to(idx.device)
        if mode == "prod":
            idx._qjl_signs = take(n, np.uint8, bpp).reshape(n, bpp).to(idx.device)
            idx._residual_norms = take(n, np.float32, 4).to(idx.device)
        idx.n_vectors = n
        return idx
