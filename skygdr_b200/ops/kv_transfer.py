"""Paged KV transfer between GPUs (and to mapped host memory).

``KvTransferFlow`` is one registered flow: a credit page, a status block and a
cumulative byte counter. ``transfer`` launches the sm_100a kernel
(skygdr_b200/csrc/kernels/kv_transfer.cu) which gathers the pages named by the
source block list, converts token-major to head-major pages, optionally packs
to block-scaled fp8, and stores into the destination pool(s) of other GPUs.
It stands where the reference calls cudaMemcpyPeerAsync
(llm_problem_analysis/kv_nvlink_transfer.cu:122,
llm_problem_analysis/kv_nvlink_transfer_trace.cu:383).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

import torch

from .._ext import load
from .flow import CreditPage, new_status, read_status
from .kv_cache import KVGeometry, PagedKVPool


@dataclass
class RemotePool:
    """A destination pool that may live on another GPU / in another process: address + geometry."""
    ptr: int
    strides: tuple          # (block, layer, kv) in destination elements
    kv_heads: int           # heads stored in this pool
    scale_ptr: int = 0      # fp8: scale bytes, same indexing / 32
    done_flag_ptr: int = 0  # optional u32 set when a transfer has fully landed
    num_blocks: int = 0     # pool size for the kernel's block-id check (0 = unchecked)

    @classmethod
    def of(cls, pool: PagedKVPool, done_flag: Optional[torch.Tensor] = None) -> "RemotePool":
        assert pool.layout == "hnd"
        return cls(pool.data.data_ptr(), pool.strides, pool.geom.kv_heads, 0,
                   done_flag.data_ptr() if done_flag is not None else 0, pool.num_blocks)


class MulticastPools:
    """Head-major pools of the same shape on every GPU of a team, all bound to one NVLink multicast object.

    ``pools[i]`` is GPU ``devices[i]``'s own copy (an ordinary ``PagedKVPool`` over that GPU's memory);
    ``multicast_ptr`` is the address whose stores NVSwitch delivers into every copy. The GPU that issues the
    stores has to be a member, so the team is the source GPU followed by the destinations and the source holds a
    copy too (the price of the fan-out: pool-sized memory on the source). One process drives all members; close()
    before the process ends so that nothing stays bound."""

    def __init__(self, geom: KVGeometry, n_blocks: int, devices: Sequence[int]):
        C = load()
        self._C = C
        self.geom, self.n_blocks, self.devices = geom, n_blocks, [int(d) for d in devices]
        for d in self.devices:
            ok, why = C.multicast_supported(d)
            if not ok:
                raise RuntimeError(f"NVLink multicast is not available on device {d}: {why}")
        elems = n_blocks * geom.block_elems
        self.region = C.multicast_create(self.devices, elems * 2)
        self.multicast_ptr = int(self.region.multicast)
        self.pools: List[PagedKVPool] = []
        shape = [n_blocks, geom.layers, 2, geom.kv_heads, geom.block_tokens, geom.head_dim]
        for i, d in enumerate(self.devices):
            data = C.tensor_from_ptr(int(self.region.unicast[i]), shape, torch.bfloat16, d)
            self.pools.append(PagedKVPool(geom, n_blocks, "hnd", data=data))

    def close(self) -> None:
        if self.region is not None:
            self.pools = []
            self._C.multicast_destroy(self.region)
            self.region = None

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


class FanoutTarget:
    """Destination pools of a 1 -> k fan-out, through the NVLink multicast address where the machine has one and as a loop of
    unicast peer stores where it has not (no NVSwitch, an old driver, a GPU outside the fabric): the caller sends the same way
    either way. ``mode`` says which was set up ("multimem" or "unicast"), ``why`` why multicast was not used."""

    def __init__(self, geom: KVGeometry, n_blocks: int, src_gpu: int, dst_gpus: Sequence[int], prefer_multicast: bool = True):
        self.geom, self.src_gpu, self.dst_gpus = geom, int(src_gpu), [int(d) for d in dst_gpus]
        self.why = ""
        self._mc: Optional[MulticastPools] = None
        if prefer_multicast and len(self.dst_gpus) >= 1:
            try:
                self._mc = MulticastPools(geom, n_blocks, [self.src_gpu] + self.dst_gpus)
            except Exception as exc:                 # capability probe or creation failed on the host: nothing ran on a GPU
                self.why = str(exc)
        if self._mc is not None:
            self.mode = "multimem"
            self.pools = self._mc.pools[1:]          # the source's own copy is not a destination
        else:
            self.mode = "unicast"
            C = load()
            for d in self.dst_gpus:
                if d != self.src_gpu and not (C.enable_peer_access(self.src_gpu, d) and C.enable_peer_access(d, self.src_gpu)):
                    raise RuntimeError(f"no peer access between GPU {self.src_gpu} and GPU {d}")
            self.pools = [PagedKVPool(geom, n_blocks, "hnd", device=torch.device("cuda", d)) for d in self.dst_gpus]
        self._remotes = [RemotePool.of(p) for p in self.pools]

    def send(self, flow: "KvTransferFlow", src: PagedKVPool, src_blocks: torch.Tensor, dst_blocks: torch.Tensor, **kw) -> None:
        """Enqueues the fan-out of ``src_blocks`` into the same ``dst_blocks`` of every destination pool."""
        if self._mc is not None:
            placeholders = [RemotePool(0, self.pools[0].strides, self.geom.kv_heads) for _ in self.pools]
            flow.transfer(src, placeholders, src_blocks, dst_blocks, replicate=True, multicast_ptr=self._mc.multicast_ptr, **kw)
        else:
            flow.transfer(src, self._remotes, src_blocks, dst_blocks, replicate=True, **kw)

    def close(self) -> None:
        self.pools, self._remotes = [], []
        if self._mc is not None:
            self._mc.close()
            self._mc = None

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


class KvTransferFlow:
    def __init__(self, device, page: Optional[CreditPage] = None, ctas: Optional[int] = None, pages_per_chunk: int = 8,
                 max_wait_ms: float = 2.0, method: str = "auto"):
        """method: "tma" (copy hardware does gather, layout change and peer write; bf16 only), "simt" (register path; also
        fp8 packing and same-layout copies), or "auto" (tma whenever it applies)."""
        assert method in ("auto", "tma", "simt")
        self.method = method
        self._ctas_given = ctas is not None
        self._C = load()
        self.device = torch.device(device)
        self.page = page
        self.status = new_status(self.device)
        self.consumed = 0
        sms = torch.cuda.get_device_properties(self.device).multi_processor_count
        self.sms = sms
        self.ctas = ctas or 2 * sms
        self.pages_per_chunk = pages_per_chunk
        self.max_wait_ns = int(max_wait_ms * 1e6)
        self.seq = 0

    def transfer(self, src: PagedKVPool, dsts: Sequence[RemotePool], src_blocks: torch.Tensor, dst_blocks: torch.Tensor,
                 replicate: bool = False, fp8: bool = False, keep_layout: bool = False, first_chunk: int = 0,
                 signal: bool = True, ctas: Optional[int] = None, multicast_ptr: int = 0) -> None:
        """Enqueues one transfer on the current stream of the source device. ``ctas`` overrides the flow's CTA count
        for this launch: a paced flow should also hold fewer SMs (its SM quota), or its waiting CTAs crowd out co-runners.
        ``multicast_ptr`` (with ``replicate``): the pages go out once through that NVLink multicast address and land in
        every team member's pool (``MulticastPools``); ``dsts`` then only names the done flags to raise."""
        assert src.layout == "nhd"
        g = src.geom
        heads_per_dst = g.kv_heads if replicate else g.kv_heads // len(dsts)
        for d in dsts:
            assert replicate or keep_layout or d.kv_heads == heads_per_dst, "destination head count does not match the scatter"
        assert not multicast_ptr or (replicate and not fp8 and not keep_layout), "multicast fan-out carries replicated bf16 pages"
        use_tma = self.method != "simt" and not multicast_ptr and not fp8 and not keep_layout and g.kv_heads <= 8 and g.head_dim == 128 and src.data.is_contiguous()
        assert use_tma or self.method != "tma", "the TMA variant moves contiguous bf16 pools of <= 8 heads without fp8 packing"
        if use_tma and ctas is None and not self._ctas_given:
            ctas = self.sms                      # one driving thread and a 192 KB ring per SM
        self.seq += 1
        self._C.reset_status(self.status)
        self._C.kv_transfer(
            src.data, [d.ptr for d in dsts], [d.scale_ptr for d in dsts], [d.done_flag_ptr if signal else 0 for d in dsts],
            src_blocks, dst_blocks, g.layers, g.kv_heads, g.block_tokens, g.head_dim, list(src.strides), list(dsts[0].strides),
            heads_per_dst, replicate, fp8, keep_layout, self.pages_per_chunk, ctas or self.ctas,
            self.page.dev_ptr if self.page else 0, self.consumed, self.max_wait_ns, first_chunk, self.seq, self.status, use_tma,
            multicast_ptr=multicast_ptr, src_num_blocks=src.num_blocks, dst_num_blocks=min(d.num_blocks for d in dsts))
        self._last = (src, dsts, src_blocks, dst_blocks, replicate, fp8, keep_layout, ctas, multicast_ptr)

    def result(self) -> Dict[str, int]:
        """Synchronises and returns the status block; accounts the bytes that were moved."""
        torch.cuda.synchronize(self.device)
        st = read_status(self.status)
        self.consumed += st["bytes_done"]
        st["device_time_ms"] = (st["t_end_ns"] - st["t_start_ns"]) * 1e-6 if st["t_end_ns"] else float("nan")
        return st

    def resume(self, st: Dict[str, int]) -> None:
        """Relaunches the last transfer from the cursor a yielded launch left behind."""
        assert st["status"] in (1, 2, 6)
        src, dsts, sb, db, rep, fp8, keep, ctas, mc = self._last
        self.transfer(src, dsts, sb, db, rep, fp8, keep, first_chunk=st["cursor"], ctas=ctas, multicast_ptr=mc)

    def transfer_to_completion(self, *args, max_launches: int = 10000, **kw) -> Dict[str, int]:
        """Transfers, relaunching after every credit yield; sums bytes and stall time."""
        self.transfer(*args, **kw)
        total = self.result()
        n = 1
        while total["status"] == 1 and n < max_launches:
            self.resume(total)
            st = self.result()
            n += 1
            for k in ("bytes_done", "chunks_done", "stall_ns"):
                st[k] += total[k]
            st["t_start_ns"] = total["t_start_ns"]
            st["device_time_ms"] = (st["t_end_ns"] - st["t_start_ns"]) * 1e-6
            total = st
        total["launches"] = n
        return total


def link_bytes(geom: KVGeometry, n_blocks: int, n_dst: int = 1, replicate: bool = False, fp8: bool = False) -> int:
    """Bytes that leave the source GPU (unicast fan-out sends every page once per destination; a multicast one, n_dst=1)."""
    per_page = geom.page_elems * (2 if not fp8 else 1) + (geom.page_elems // 32 if fp8 else 0)
    return n_blocks * geom.layers * 2 * per_page * (n_dst if replicate else 1)


def reference_transfer(src: PagedKVPool, src_blocks: torch.Tensor, heads: slice = slice(None)) -> torch.Tensor:
    """What a destination pool's blocks must hold after a transfer: [n][layer][2][head][tok][dim]."""
    x = src.data[src_blocks.long()]            # [n][L][2][T][H][D]
    return x.permute(0, 1, 2, 4, 3, 5)[:, :, :, heads].contiguous()


def fp8_mx_reference(x: torch.Tensor):
    """Block-scaled e4m3 packing of the last dim in groups of 32: returns (fp8 bytes as uint8, scale bytes)."""
    shp = x.shape
    g = x.float().reshape(*shp[:-1], shp[-1] // 32, 32)
    amax = g.abs().amax(-1, keepdim=True)
    mant, exp = torch.frexp(amax)               # amax = mant * 2^exp, mant in [0.5, 1)
    e = (exp - 1 - 8 + (mant > 0.875).to(exp.dtype)).float()   # smallest e with amax / 2^e <= 448 = 1.75 * 2^8
    e = torch.where(amax > 0, e, torch.full_like(e, -127.0)).clamp(-127, 127)
    q = (g * torch.exp2(-e)).to(torch.float8_e4m3fn)
    return q.view(torch.uint8).reshape(shp), (e + 127).to(torch.uint8).reshape(*shp[:-1], shp[-1] // 32)
