"""The bfloat16 serving kernels: tensor-core products (and tiled attention).

Each call returns ``True`` if it ran and ``False`` if the kernel refuses the
sizes (the caller then uses the any-size kernel).  Refusal is decided on the
host from the kernel's stated limits, never by trying.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_longlong, c_void_p, byref

import torch

from ..csrc.build import ensure_built


def _ptr(t):
    return c_void_p(0 if t is None else t.data_ptr())


class FastKernels:
    def __init__(self, device):
        self.device = torch.device(device)
        self.lib = ctypes.CDLL(ensure_built("bf16"))
        self.sm_count = torch.cuda.get_device_properties(self.device).multi_processor_count
        self._configure()
        self.lib.leone_attention_decode_scratch.restype = ctypes.c_longlong
        self.lib.leone_gemm_pair_workspace_floats.restype = ctypes.c_longlong

    def _configure(self) -> None:
        """The switches and rules of the dispatchers (everything but the device and the library)."""
        self._workspace = None
        self._retired = []
        self.min_scratch_floats = 1 << 20
        self._counters = None
        # LEONE_NO_TENSOR_CORES=1 routes every product to the CUDA-core kernel (for fault finding)
        self.use_tensor_cores = os.environ.get("LEONE_NO_TENSOR_CORES", "0") != "1"
        # LEONE_NO_CLUSTERS=1 sums split-K partial tiles through a workspace instead of inside clusters
        self.use_clusters = os.environ.get("LEONE_NO_CLUSTERS", "0") != "1"
        self._cluster_capacity = {}
        # LEONE_NO_FUSED_NORM=1 keeps every RMSNorm a kernel of its own
        self.fuse_norm = os.environ.get("LEONE_NO_FUSED_NORM", "0") != "1"
        self.fuse_norm_tokens = 32
        # LEONE_NO_TOKEN_MAJOR=1 keeps every product of up to 256 tokens in the swapped form
        # LEONE_NO_DIVIDED_STEPS=1 sends a mixed step's decode rows through the prompt attention kernel too
        self.divide_mixed_steps = os.environ.get("LEONE_NO_DIVIDED_STEPS", "0") != "1"
        self.mixed_decode_rows_from = 1
        self.use_token_major = os.environ.get("LEONE_NO_TOKEN_MAJOR", "0") != "1"
        self.token_major_from = 64         # tokens above which the token-major form is considered
        self.token_major_split_from = 128  # .. and its split along K (up to 128 tokens the swapped form's split measured the same or better)
        self.token_major_fill = 0.6        # of the SMs that its tiles must fill
        self.force_decode_splits = 0       # > 0: every decode attention splits its keys this many ways (kernel_bench sets it)
        # LEONE_NO_FUSED_DECODE=1 keeps q/k norm, rotation and cache write in their own kernel
        self.fuse_decode = os.environ.get("LEONE_NO_FUSED_DECODE", "0") != "1"
        self.max_cluster = 8               # the portable cluster size
        # LEONE_NO_PAIRS=1 keeps prompt-sized products on single SMs (cta_group::1)
        self.use_pairs = os.environ.get("LEONE_NO_PAIRS", "0") != "1"
        self.pairs_from = 129              # tokens from which unsplit products run on pairs
        # LEONE_NO_PAIR_SPLITS=1 leaves the narrow products' split along K to the single-block kernel
        self.use_pair_splits = os.environ.get("LEONE_NO_PAIR_SPLITS", "0") != "1"
        self.pair_padding = 0.8            # a pair's half tile against a single block's tile, at most (see in_pairs)
        self.pair_width_override = 0       # > 0: the tile width of every product on pairs (kernel_bench sets it)
        self.pair_split_override = 0       # > 0: pairs per tile of every product on pairs (tests set it)
        self._pair_widths = {}
        self._plans = {}                   # _gemm's decisions per (sizes, arguments)
        self.decode_cluster_rounds = 1     # rounds of blocks a clustered decode attention may take (kernel_bench sets it)
        # (n, k) -> (splits, cluster): a forced split of an [n x k] product at decode sizes; empty
        # in the product, filled by kernel_bench's sweeps
        self.split_override = {}
        self.status = None
        self._attn_ws = None
        self._pinned_stream = None
        self.use_tiled_attention = os.environ.get("LEONE_NO_TILED_ATTENTION", "0") != "1"
        # LEONE_NO_TC_ATTENTION=1 keeps prompt attention on the mma.sync kernel
        self.use_tc_attention = os.environ.get("LEONE_NO_TC_ATTENTION", "0") != "1"

    def __setattr__(self, name, value):
        # a switch changed (a test, the kernel bench): the remembered decisions may no longer hold
        if not name.startswith("_") and "_plans" in self.__dict__:
            self._plans.clear()
            self._pair_widths.clear()
        object.__setattr__(self, name, value)

    def _stream(self):
        if self._pinned_stream is not None:        # (a handle of 0, the default stream, is a valid pin)
            return self._pinned_stream
        return c_void_p(torch.cuda.current_stream(self.device).cuda_stream)

    def pin_stream(self, handle) -> None:
        """The stream every launch goes to until ``pin_stream(None)``: a step looks its stream up
        once, not once per launch (the lookup costs microseconds, a step has hundreds of launches)."""
        object.__setattr__(self, "_pinned_stream", handle)

    # -- split-K scratch ----------------------------------------------------------------
    def _retire(self, tensor) -> None:
        """A scratch buffer that is outgrown is kept, not freed: a captured CUDA graph may have
        its address baked in and will go on using it."""
        if tensor is not None:
            self._retired.append(tensor)

    def token_major_workspace_floats(self) -> int:
        """One 128 x 256 fp32 partial tile per block of a round."""
        return self.sm_count * 128 * 256

    def scratch_bytes(self) -> int:
        """What these ops allocate for themselves at most: the split products' workspace and the
        split decode attention's partial results."""
        return 4 * (max(self.min_scratch_floats, self.token_major_workspace_floats()) + self.min_scratch_floats)

    def _scratch(self, floats: int, counters: int):
        if self._workspace is None or self._workspace.numel() < floats:
            self._retire(self._workspace)
            self._workspace = torch.empty(max(floats, self.min_scratch_floats), dtype=torch.float32,
                                          device=self.device)
        if self._counters is None or self._counters.numel() < counters:
            self._retire(self._counters)
            self._counters = torch.zeros(max(counters, 4096), dtype=torch.int32, device=self.device)
        return self._workspace, self._counters

    def cluster_capacity(self, m: int, splits: int) -> int:
        """Clusters of ``splits`` blocks of the GEMM for ``m`` tokens that fit on the device at once."""
        key = (int(self.lib.leone_gemm_tc_tile(m)) if m <= 256 else 0, splits)
        if key not in self._cluster_capacity:
            self._cluster_capacity[key] = int(self.lib.leone_gemm_tc_cluster_capacity(m, splits))
        return self._cluster_capacity[key]

    def choose_splits(self, m: int, n: int, k: int):
        """How to split K: ``(splits, full_tiles, cluster)``; tiles before ``full_tiles`` are not split.

        Fewer tiles than SMs: every tile is split, and its splits form a thread-block cluster that
        sums the partial tiles through distributed shared memory.  The most splits (up to 8) win
        that keep the blocks within two thirds of the block slots: more blocks keep more bytes in
        flight, but the last third is what lets the next kernels' blocks start early and fetch
        their first weights while this product is still running (measured on the decode step:
        filling every slot was slower than leaving the product unsplit).  More tiles than SMs:
        only a small remainder of tiles (under a quarter of the SMs) is split, through a
        workspace, so that those few tiles do not cost a round of their own; such a unit keeps
        at least 12 k-blocks.  Prompt-sized M is never split."""
        tiles = int(self.lib.leone_gemm_tc_tiles(m, n))
        if m > 256:
            return 1, tiles, False
        k_blocks = -(-k // 64)
        sms = self.sm_count
        if (n, k) in self.split_override:
            s, cluster = self.split_override[(n, k)]
            return (s, 0, cluster) if s > 1 else (1, tiles, False)
        if tiles < sms:
            slots = sms * (2 if m <= 64 else 1)
            if self.use_clusters:
                for s in (8, 7, 6, 5, 4, 3, 2):
                    if tiles * s <= slots * 2 // 3 and k_blocks // s >= 4 and s <= self.max_cluster and self.cluster_capacity(m, s) > 0:
                        return s, 0, True
            s = max(1, min(sms // tiles, k_blocks // 12, 8))
            return (s, 0, False) if s > 1 else (1, tiles, False)
        rem = tiles % sms
        if rem == 0 or rem * 4 > sms:
            return 1, tiles, False
        s = min(sms // rem, k_blocks // 12, 8)
        return (s, tiles - rem, False) if s > 1 else (1, tiles, False)

    def _tc_ok(self, x, w, out) -> bool:
        if not self.use_tensor_cores or x.dtype != torch.bfloat16:
            return False
        k = x.shape[1]
        return (k % 8 == 0 and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0
                and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)

    def token_major(self, m: int, n: int) -> bool:
        """Which form of the product runs: tokens on the MMA's 128-row side and 256 weight rows
        per tile (True), or weights on that side and the tokens as the tile's width (False).
        Always above 256 tokens.  From 65 to 256 tokens too when the token-major tiles fill
        at least ``token_major_fill`` of the SMs and at most two rounds of them (the gate/up
        product of a wide feed-forward): the swapped form re-reads the whole token operand for
        every 128 weight rows, twice the bytes of the weights at 256 tokens (gate/up of the 8B
        shape: 65 µs against 49 at 128 tokens, 100 against 68 at 256).  With fewer tiles the
        swapped form's split along K keeps more SMs busy; with many more (an output head, whose
        time is the fp32 logits it writes) the swapped form measured a few percent faster."""
        if m > 256:
            return True
        if m <= self.token_major_from or not self.use_token_major:
            return False
        tiles = int(self.lib.leone_gemm_tc_tiles_token_major(m, n))
        return self.token_major_fill * self.sm_count <= tiles <= 2 * self.sm_count

    def in_pairs(self, m: int, n: int = 0, k: int = 0) -> bool:
        """Whether an unsplit product of ``m`` tokens runs on pairs of SMs (tiles of 256 tokens,
        the width chosen by :meth:`pair_width`): from 129 tokens on, except from 257 to 384
        tokens, where the second of two tiles of 256 would be half empty and the single-block
        kernel's three tiles of 128 measured faster (gate/up at 384 tokens 62.3 us against 67.2;
        at 640 tokens three pairs already beat five single tiles, 95.9 against 105.6).  With
        ``n`` and ``k``: whether this ``[n x k]`` product does; the narrow products of a layer,
        which up to about 600 tokens are split along K, do not (with tiles narrow enough to fill
        the pairs, all pairs read the same few token tiles at once, and that measured slower
        than the split: o_proj at 256 tokens 25.3 us against 18.7, down 61.7 against 37.1)."""
        if n and k and self.token_major_split(m, n, k) > 1:
            return self.pair_split(m, n, k) > 1
        return self._pairs_fit(m)

    def _pairs_fit(self, m: int) -> bool:
        return self.use_pairs and m >= self.pairs_from and 2 * -(-m // 256) * self.pair_padding <= -(-m // 128)

    def pair_split(self, m: int, n: int, k: int) -> int:
        """Pairs of SMs per tile of a narrow product (one that the single-block kernel would split
        along K): 4 or 2 pairs share the k-blocks of a tile of 256 tokens x 256 weight rows when
        their clusters of 8 or 4 blocks are all resident at once and a pair keeps at least 8
        k-blocks; 1: not split on pairs.  Only where the pairs can split as many ways as the single
        blocks would: with the same number of splits the pairs' k-loop wins (down at 512 tokens
        50.3 us against 56.6, qkv at 256 tokens 23.4 against 25.3), against four single-block
        splits two pairs lose (o_proj at 256 tokens 25.1 us against 18.8, down 46.5 against 37.4).
        Also from 257 to 384 tokens, where unsplit products stay in single blocks (down at 320
        tokens 48.6 us against 55.4)."""
        if self.pair_split_override:
            return self.pair_split_override
        if not (self.use_pair_splits and self.use_clusters and self.use_pairs and m >= self.pairs_from) or \
                self.token_major_split(m, n, k) == 1:
            return 1
        tiles, k_blocks = -(-n // 256) * -(-m // 256), -(-k // 64)
        single = self.token_major_split(m, n, k)
        for s in (4, 2):
            if tiles * s <= self.sm_count // 2 and k_blocks // s >= 8 and tiles <= self._pair_capacity(s):
                return s if s >= single else 1
        return 1

    def _pair_capacity(self, splits: int) -> int:
        key = ("pairs", splits)
        if key not in self._cluster_capacity:
            self._cluster_capacity[key] = int(self.lib.leone_gemm_pair_capacity(256, splits))
        return self._cluster_capacity[key]

    def pair_width(self, m: int, n: int, swiglu: bool) -> int:
        """Weight rows per tile of a product on pairs of SMs: the width whose tiles cost the
        fewest rounds over the pairs.  A tile's k-block costs what the copy of its operands
        into a block's shared memory takes (128 token rows beside width / 2 weight rows: the
        k-loop runs at the rate of those copies, 32 KB in 0.36 us, at every width that was
        measured); of two widths within 1 percent the wider one stays."""
        if self.pair_width_override:
            return self.pair_width_override
        key = (-(-m // 256), n, bool(swiglu))
        if key not in self._pair_widths:
            pairs, best = self.sm_count // 2, None
            for w in range(256, 31, -32 if swiglu else -16):
                rounds = -(-(-(-n // w) * key[0]) // pairs)
                cost = rounds * (0.18 + 0.0007 * w)
                if best is None or cost < 0.99 * best[0]:
                    best = (cost, w)
            self._pair_widths[key] = best[1]
        return self._pair_widths[key]

    def token_major_split(self, m: int, n: int, k: int) -> int:
        """Splits along K of the token-major form, summed inside thread-block clusters (1: none).
        A product whose token-major tiles fill at most half of the SMs (the narrow products of a
        layer between 65 and about 600 tokens) is split so that tiles x splits blocks fill them;
        a split keeps at least 8 k-blocks.  Such a product takes no folded norm."""
        if not (self.use_clusters and self.use_token_major) or m <= self.token_major_split_from:
            return 1
        tiles = int(self.lib.leone_gemm_tc_tiles_token_major(m, n))
        if tiles * 2 > self.sm_count:
            return 1
        k_blocks = -(-k // 64)
        # all clusters must be resident at once: a cluster needs its blocks' SMs free in one GPC
        # at the same moment, and a grid that needs a second round of clusters was measured at
        # twice the time (the occupancy query's count of resident clusters is what holds)
        for s in range(min(8, self.sm_count // tiles, self.max_cluster), 1, -1):
            if k_blocks // s >= 8 and tiles <= self._token_major_capacity(s):
                return s
        return 1

    def _token_major_capacity(self, splits: int) -> int:
        key = ("token-major", splits)
        if key not in self._cluster_capacity:
            self._cluster_capacity[key] = int(self.lib.leone_gemm_tc_cluster_capacity_token_major(splits))
        return self._cluster_capacity[key]

    def plan_product(self, m: int, n: int, k: int):
        """``(token_major, splits, full_tiles, cluster)`` for a product without a folded norm."""
        if self.in_pairs(m, n, k):
            return True, 1, 0, False                 # on pairs of SMs (_gemm takes them where nothing is forced)
        s = self.token_major_split(m, n, k)
        if s > 1:
            return True, s, 0, True
        if self.token_major(m, n):
            return True, 1, 0, False
        return (False, *self.choose_splits(m, n, k))

    def _gemm(self, x, w, out, epilogue, residual, n_rows, splits=None, full_tiles=0, cluster=False,
              norm_in=None, norm_out=None, token_major=None) -> bool:
        """``splits=None`` lets :meth:`choose_splits` decide; otherwise tiles from
        ``full_tiles`` on are split ``splits`` ways, summed through a workspace or, with
        ``cluster``, inside a thread-block cluster.

        ``norm_out=(xn, weight, ss)``: the product (fp32 output) also leaves
        ``xn = bf16(out * weight)`` and the partial sums of ``out^2`` in ``ss`` ``[parts, m]``
        for the RMSNorm that follows it; ``norm_in=(ss, parts, eps)``: ``x`` is such an ``xn``
        and every output row is scaled by the norm's ``rsqrt(mean + eps)``."""
        m, k = x.shape
        key = (m, n_rows, k, epilogue, splits, full_tiles, cluster, token_major, norm_in is not None,
               norm_out is not None)
        plan = self._plans.get(key)
        if plan is None:
            plan = self._plans[key] = self._plan_gemm(*key)
        pairs, token_major, splits, full_tiles, cluster, ws_floats, ws_counters, parts, width = plan
        ws = ct = None
        if ws_floats or ws_counters:
            ws, ct = self._scratch(ws_floats, ws_counters)
            if not ws_counters:
                ct = None
        if norm_out is not None and norm_out[2].shape[0] != parts:
            raise ValueError(f"the sums of squares have {norm_out[2].shape[0]} parts, this product leaves {parts}")
        no = (None, None, None, 0) if norm_out is None else \
            (_ptr(norm_out[0]), _ptr(norm_out[1]), _ptr(norm_out[2]), norm_out[0].stride(0))
        ni = (None, 0, c_float(0.0)) if norm_in is None else (_ptr(norm_in[0]), int(norm_in[1]), c_float(norm_in[2]))
        if pairs:
            # pairs of SMs on tiles of 256 tokens (gemm_pair.cu)
            code = self.lib.leone_gemm_pair(_ptr(x), _ptr(w), _ptr(out), _ptr(residual), m, n_rows, k,
                                            x.stride(0), w.stride(0), out.stride(0), epilogue, width, splits, _ptr(ws),
                                            _ptr(self.status), self.sm_count, *no, *ni, self._stream())
            if code != 0:
                raise RuntimeError(f"gemm_pair refused or failed with code {code} for m={m} n={n_rows} k={k}")
            return True
        code = self.lib.leone_gemm_tc(_ptr(x), _ptr(w), _ptr(out), _ptr(residual), m, n_rows, k,
                                      x.stride(0), w.stride(0), out.stride(0), epilogue, splits,
                                      full_tiles, _ptr(ws), _ptr(ct), _ptr(self.status), self.sm_count,
                                      1 if cluster else 0, 1 if token_major else 0, *no, *ni, self._stream())
        if code != 0:
            raise RuntimeError(f"gemm_tc refused or failed with code {code} for m={m} n={n_rows} k={k} "
                               f"splits={splits} cluster={cluster} token_major={token_major}")
        return True

    def _plan_gemm(self, m, n_rows, k, epilogue, splits, full_tiles, cluster, token_major, has_norm_in, has_norm_out):
        """What :meth:`_gemm` does for one combination of sizes and arguments (kept per combination;
        every change of a switch of this object forgets the plans): ``(pairs, token_major, splits,
        full_tiles, cluster, workspace floats, counters, parts of a folded norm's sums, tile width
        on pairs)``.  On pairs, ``splits`` is the number of pairs per tile."""
        no_norm = not has_norm_in and not has_norm_out
        # on pairs of SMs unless the caller forces another form
        pairs = token_major is None and splits in (None, 1) and not cluster and self.in_pairs(m, n_rows, k)
        if pairs:
            ps = self.pair_split(m, n_rows, k) if no_norm else 1
            width, floats = self.pair_width(m, n_rows, epilogue == 3), 0
            if ps > 1:
                width = 256
                floats = max(self.token_major_workspace_floats(),
                             int(self.lib.leone_gemm_pair_workspace_floats(m, n_rows, width, ps)))
            return True, True, ps, 0, False, floats, 0, self.norm_parts(m, n_rows, True), width
        if token_major is None and splits is None and no_norm:
            token_major, splits, full_tiles, cluster = self.plan_product(m, n_rows, k)
        token_major = bool(token_major) or m > 256
        if token_major and not cluster:
            splits, full_tiles = 1, 0
        elif splits is None:
            splits, full_tiles, cluster = self.choose_splits(m, n_rows, k)
        floats = counters = 0
        if splits > 1 and not cluster:
            tiles = int(self.lib.leone_gemm_tc_tiles(m, n_rows))
            f, c = c_longlong(0), c_int(0)
            self.lib.leone_gemm_tc_scratch(m, max(tiles - full_tiles, 0), splits, byref(f), byref(c))
            floats, counters = f.value, c.value
        elif splits > 1 and token_major:
            # the token-major form's partial tiles (128 tokens x 256 weight rows, fp32) cross
            # between the blocks of a cluster through the workspace
            # (one round of blocks at most, so the largest request is asked for at once and the
            # buffer never grows with the step's size)
            floats = self.token_major_workspace_floats()
        return False, token_major, splits, full_tiles, bool(cluster), floats, counters, \
            self.norm_parts(m, n_rows, False), 0

    def fuses_norm(self, m: int, n: int = 0, k: int = 0) -> bool:
        """Whether the products of ``m`` tokens carry an RMSNorm between them: decode-sized steps
        (up to 32 tokens; from there to 256 the extra work in the two epilogues was measured to
        cost more than the norm kernel it replaces) and prompt-sized ones (over 256 tokens,
        where a thread owns a token row and the sums are its own).  With ``n`` and ``k``: whether
        this ``[n x k]`` product does; one that is split in the token-major form does not."""
        if not (self.use_tensor_cores and self.fuse_norm and (0 < m <= self.fuse_norm_tokens or m > 256)):
            return False
        return not (n and k and self.token_major_split(m, n, k) > 1)

    def norm_parts(self, m: int, n: int, pairs=None) -> int:
        """Parts of the sums of squares that a product of ``m`` tokens with ``n`` outputs leaves
        for the norm after it: on pairs of SMs (``pairs=None``: where the dispatcher takes them
        for an unsplit product) one per tile of weight rows, else what the single-block kernel
        leaves."""
        if self.in_pairs(m) if pairs is None else pairs:
            return -(-n // self.pair_width(m, n, False))
        return int(self.lib.leone_gemm_tc_norm_parts(m, n))

    def linear(self, x, w, out, epilogue, residual, norm_in=None, norm_out=None) -> bool:
        if not self._tc_ok(x, w.weight, out):
            return False
        return self._gemm(x, w.weight, out, epilogue, residual, w.out_features, norm_in=norm_in, norm_out=norm_out)

    # -- gate/up --------------------------------------------------------------------------
    def prepare_gate_up(self, gate, up):
        from .cuda import PreparedMatrix
        inter, hidden = gate.shape
        if gate.dtype == torch.bfloat16 and inter % 16 == 0 and hidden % 8 == 0 and self.use_tensor_cores:
            # groups of 32 rows: 16 gate rows, then the 16 up rows of the same columns
            stacked = torch.stack([gate.view(inter // 16, 16, hidden), up.view(inter // 16, 16, hidden)],
                                  dim=1).reshape(2 * inter, hidden).contiguous()
            m = PreparedMatrix(stacked)
            m.gate_up_layout = "interleaved16"
            return m
        m = PreparedMatrix(torch.cat([gate, up], dim=0).contiguous())
        m.gate_up_layout = "stacked"
        return m

    def linear_swiglu(self, x, w, out, norm_in=None) -> bool:
        if getattr(w, "gate_up_layout", None) != "interleaved16" or not self._tc_ok(x, w.weight, out):
            return False
        return self._gemm(x, w.weight, out, 3, None, w.out_features, norm_in=norm_in)

    # -- attention ------------------------------------------------------------------------
    def decode_splits(self, n_seqs: int, n_kv: int, g: int, max_ctx: int) -> int:
        """Splits of the key range.  Two blocks fit an SM; the cost of a choice is its number of
        rounds over those slots times the share of the keys a block walks, plus a little per
        split for the merge (since the partial results are pushed into the finishing block the
        merge costs next to nothing: batch 1 at 2,048 keys 9.7 / 9.1 / 8.6 us for six / seven /
        eight splits, at 16,384 keys 50 / 39 us for six / eight), plus a fixed charge when the
        splits cannot merge inside clusters
        (scratch, a merge kernel and the q/k preparation in a kernel of its own: a fixed part,
        measured at batch 64: one split 101 us, two to four 109-112, and at batch 20: one fused
        split 50.0 us, seven splits 52.1; and a fifth of the walk, measured at batches 160 to 224:
        one fused split 242 / 289 / 326 us, three to six splits 250 / 309 / 366; at batch 48
        three splits are still the better choice, 91 us against 97).  The fixed parts were
        measured at 2,048 keys and are so many microseconds whatever the context, so in units of
        a walk they shrink as the context grows: at batch 1 sixteen to thirty-two unclustered
        splits beat eight clustered ones from 16,384 keys on (33 against 40 us; at 32,768 keys 46
        against 75), at 8,192 keys they do not (24.5 against 22.4); the share of the walk shrinks
        too, with the root of that factor (a short block's own start and end are what it stands
        for: batch 16 at 32,768 keys, nine unclustered splits 351 us against 378 for two
        clustered ones).  A split keeps at least 128 keys."""
        if self.force_decode_splits:
            return self.force_decode_splits
        blocks = n_seqs * n_kv * (-(-g // 16))
        slots = 2 * self.sm_count
        best, best_cost = 1, None
        fixed = 2048.0 / max(max_ctx, 128)        # the charges that do not grow with the keys, in walks
        for s in range(1, min(32, max(1, max_ctx // 128)) + 1):
            clustered = self.use_clusters and s <= 8 and blocks * s <= self._decode_cluster_slots()
            walk = -(-(blocks * s) // slots) / s
            cost = walk + fixed * (0.01 * s + (0.0 if s == 1 or clustered else 0.3)) + \
                (0.0 if s == 1 or clustered else 0.2 * fixed ** 0.5 * walk)
            if best_cost is None or cost < best_cost - 1e-9:
                best, best_cost = s, cost
        return best

    def attention_supported(self, dtype, n_q, n_kv, d, row_stride) -> bool:
        return (self.use_tiled_attention and dtype == torch.bfloat16 and d % 16 == 0 and d <= 128
                and n_q // n_kv <= 64 and row_stride % 8 == 0)

    def decode_fusable(self, ctx, dtype, n_q, n_kv, d, row_stride) -> bool:
        """True if a decode step's attention runs as clusters that can also do the q/k norm,
        the rotation and the cache write."""
        return (self.attention_supported(dtype, n_q, n_kv, d, row_stride) and self.fuse_decode
                and ctx.decode_only and d in (64, 128)
                and self.decode_in_clusters(ctx.n_seqs, n_kv, n_q // n_kv, ctx.max_ctx_len))

    def decode_in_clusters(self, n_seqs: int, n_kv: int, g: int, max_ctx: int) -> bool:
        """Whether a decode step runs the kernel whose splits merge inside thread-block clusters
        (and which can do the q/k preparation itself): with one split, or when all blocks are
        resident at once.  With several rounds of blocks, clusters (which need all their
        blocks' slots free in one GPC at the same moment) were measured slower than scratch
        and a merge kernel."""
        splits = self.decode_splits(n_seqs, n_kv, g, max_ctx)
        blocks = n_seqs * n_kv * (-(-g // 16)) * splits
        return self.use_clusters and (splits == 1 or (splits <= 8 and blocks <= self._decode_cluster_slots()))

    def _decode_cluster_slots(self) -> int:
        """Blocks of the decode attention that clusters may count on at once: nine tenths of the
        two per SM (a cluster needs its blocks' slots in one GPC, and the GPCs are not all the same
        size: 96 clusters of three, 288 of 296 slots, measured 42.7 us at batch 12 where 96
        clusters of two take 33.9 us; 64 clusters of four, 256 slots, are the best choice at
        batch 8)."""
        return 2 * self.sm_count * 9 // 10 * self.decode_cluster_rounds

    def leading_decode_rows(self, ctx) -> int:
        """In a mixed step, how many sequences at the front of the batch bring a single token
        (the scheduler puts decode rows first).  Their attention runs on the decode kernel
        (which streams a sequence's keys once for all its heads) and the rest on the prompt
        kernel, which would spend a 128-row tile on each of them.  0: do not divide the step."""
        q_lens = getattr(ctx, "q_lens", None)
        if ctx.decode_only or getattr(ctx, "fixed_shapes", False) or q_lens is None or not self.divide_mixed_steps:
            return 0
        n = 0
        while n < len(q_lens) and q_lens[n] == 1:
            n += 1
        return n if self.mixed_decode_rows_from <= n < len(q_lens) else 0

    def attention(self, ctx, qkv, out, n_q, n_kv, d, scale, window, cache, fuse=None) -> bool:
        if not self.attention_supported(qkv.dtype, n_q, n_kv, d, qkv.stride(0)):
            return False
        bt = cache.block_table
        args = (qkv, out, n_q, n_kv, d, scale, window, cache)
        if ctx.decode_only:
            self._attention_decode(*args, ctx.q_start, ctx.ctx_len, bt, ctx.n_seqs, ctx.max_ctx_len, ctx.status, fuse)
            return True
        if fuse is not None:
            raise RuntimeError("fused q/k preparation is a decode-step feature")
        n_dec = self.leading_decode_rows(ctx)
        if n_dec:
            self._attention_decode(*args, ctx.q_start[:n_dec + 1], ctx.ctx_len[:n_dec], bt[:n_dec], n_dec,
                                   int(ctx.ctx_lens[:n_dec].max()), ctx.status, None)
        self._attention_prompt(*args, ctx.q_start[n_dec:], ctx.ctx_len[n_dec:], bt[n_dec:], ctx.n_seqs - n_dec,
                               int(ctx.q_lens[n_dec:].max()) if n_dec else ctx.max_q_len, ctx.status)
        return True

    def _attention_decode(self, qkv, out, n_q, n_kv, d, scale, window, cache, q_start, ctx_len, bt, n_seqs,
                          max_ctx, status, fuse) -> None:
        """Sequences with one query token each (row ``q_start[s]``)."""
        from ctypes import c_float
        g = n_q // n_kv
        kp, vp = cache.k_pool, cache.v_pool
        common = (_ptr(qkv), qkv.stride(0), _ptr(out), out.stride(0), _ptr(kp), _ptr(vp), _ptr(bt),
                  bt.stride(0), _ptr(q_start), _ptr(ctx_len), n_seqs)
        splits = self.decode_splits(n_seqs, n_kv, g, max_ctx)
        if self.decode_in_clusters(n_seqs, n_kv, g, max_ctx):
            # the splits of a (sequence, KV head) merge inside a cluster; optionally the
            # kernel norms and rotates q and the new k and writes the cache itself
            fz = (0, None, None, c_float(0.0), None, 0, 0, 0)
            if fuse is not None:
                rope = fuse["rope"]
                fz = (1, _ptr(fuse["q_w"]), _ptr(fuse["k_w"]), c_float(fuse["eps"]), _ptr(rope),
                      rope.shape[0] if rope is not None else 0, 1 if fuse["write_cache"] else 0,
                      1 if fuse.get("pairing", "half_split") == "adjacent" else 0)
            code = self.lib.leone_attention_decode_cluster(
                *common, n_q, n_kv, d, c_float(scale), int(window or 0), cache.page_tokens,
                kp.shape[0], splits, *fz, _ptr(status), self._stream())
        else:
            if fuse is not None:
                raise RuntimeError("fused decode attention asked for where decode_fusable() is false")
            scratch = None
            if splits > 1:
                need = self.lib.leone_attention_decode_scratch(n_seqs, n_q, d, splits)
                scratch = self._attn_scratch(need)
            code = self.lib.leone_attention_decode(
                *common, n_q, n_kv, d, c_float(scale), int(window or 0), cache.page_tokens,
                kp.shape[0], splits, _ptr(scratch), _ptr(status), self._stream())
        if code != 0:
            raise RuntimeError(f"decode attention refused or failed with code {code}")

    def _attention_prompt(self, qkv, out, n_q, n_kv, d, scale, window, cache, q_start, ctx_len, bt, n_seqs,
                          max_q_len, status) -> None:
        """Sequences with any number of query tokens (rows ``q_start[s] .. q_start[s + 1]``)."""
        from ctypes import c_float
        g = n_q // n_kv
        kp, vp = cache.k_pool, cache.v_pool
        # head sizes 64 and 128 run on tcgen05; the others on the mma.sync kernel
        tc = self.use_tc_attention and d in (64, 128) and g <= 128 and out.stride(0) % 8 == 0
        entry = self.lib.leone_attention_prefill_pingpong if tc else self.lib.leone_attention_prefill
        code = entry(_ptr(qkv), qkv.stride(0), _ptr(out), out.stride(0), _ptr(kp), _ptr(vp), _ptr(bt),
                     bt.stride(0), _ptr(q_start), _ptr(ctx_len), n_seqs, max_q_len, n_q, n_kv, d,
                     c_float(scale), int(window or 0), cache.page_tokens, kp.shape[0], _ptr(status),
                     self._stream())
        if code != 0:
            raise RuntimeError(f"prompt attention refused or failed with code {code}")

    def _attn_scratch(self, floats: int):
        if self._attn_ws is None or self._attn_ws.numel() < floats:
            self._retire(self._attn_ws)
            self._attn_ws = torch.empty(max(floats, self.min_scratch_floats), dtype=torch.float32,
                                        device=self.device)
        return self._attn_ws
