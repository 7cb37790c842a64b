"""Weights of a training job (Megatron-style tensor / pipeline / expert parallel shards) handed to an inference engine
with another tensor-parallel layout, tensor by tensor, without ever assembling a full copy on one rank.

    specs  = decoder_specs(num_layers=.., hidden=.., ffn=.., heads=.., kv_heads=.., head_dim=.., vocab=..)
    job    = TrainToInferResharder(specs, TrainLayout(tp=4, pp=2), InferLayout(tp=2, ranks=[0, 1]), rank, executor)
    for name, shard in job.per_tensor(local_state_dict):      # on every rank; yields on the inference ranks only
        engine.load_weight(name, shard)                       # this rank's tensor-parallel slice, inference naming

What it takes care of, and what the reference's VeRL -> SGLang preprocessor does with the same planner
(app/tensorRTL/examples/verl/rl_reshard_preprocessor.py:34-700, model_adaptor/qwen_adaptor.py):
  * naming: every parameter has a training name and one or more inference names;
  * fused parameters: a training shard of linear_qkv / linear_fc1 is a concatenation of blocks (q, k, v per query
    group; gate, up) that are sharded separately, so each block is planned as a tensor of its own and the inference side
    gets them per block or re-fused in its own order;
  * pipeline stages: a layer's tensors live on the tensor-parallel ranks of its stage only;
  * experts: expert e lives on one expert-parallel group of its stage (optionally sharded inside it) and goes either to
    every inference rank (tensor-parallel experts) or to the inference rank that owns it (expert-parallel inference);
  * buckets: tensors move in buckets of bounded size through one executor call each, so the receive buffers of one
    bucket are all that is alive beside the model.
The plan is a pure function of the specs and the two layouts: every rank computes the same task lists."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Iterator, List, Optional, Sequence, Tuple

import torch

from .plan import PTensor, PTensorSet, shard_bounds


@dataclass
class TrainLayout:
    """ranks[p * tp + t] is the global rank of pipeline stage p, tensor-parallel rank t (data-parallel replica 0: the
    replicas hold the same weights and take no part). Experts of a stage are spread over ``ep`` groups of tp / ep ranks."""
    tp: int
    pp: int = 1
    ep: int = 1
    ranks: Optional[Sequence[int]] = None

    def __post_init__(self):
        if self.ranks is None:
            self.ranks = list(range(self.tp * self.pp))
        if len(self.ranks) != self.tp * self.pp:
            raise ValueError(f"{len(self.ranks)} ranks for tp {self.tp} x pp {self.pp}")
        if self.tp % self.ep != 0:
            raise ValueError("the expert-parallel size must divide the tensor-parallel size of a stage")

    def stage_ranks(self, stage: int) -> List[int]:
        return list(self.ranks[stage * self.tp:(stage + 1) * self.tp])

    def stage_of_layer(self, layer: int, num_layers: int) -> int:
        per = (num_layers + self.pp - 1) // self.pp
        return min(layer // per, self.pp - 1)

    def expert_ranks(self, stage: int, expert: int, num_experts: int) -> List[int]:
        etp = self.tp // self.ep
        g = expert // (num_experts // self.ep)
        return self.stage_ranks(stage)[g * etp:(g + 1) * etp]


@dataclass
class InferLayout:
    """Inference engine: tensor parallel over ``ranks``; ``ep`` = len(ranks) places whole experts on their owner rank,
    ep = 1 shards every expert over all ranks like a dense layer."""
    tp: int
    ranks: Optional[Sequence[int]] = None
    ep: int = 1

    def __post_init__(self):
        if self.ranks is None:
            self.ranks = list(range(self.tp))
        if len(self.ranks) != self.tp:
            raise ValueError(f"{len(self.ranks)} ranks for tp {self.tp}")
        if self.ep not in (1, self.tp):
            raise ValueError("inference experts are either tensor parallel (ep = 1) or one group per rank (ep = tp)")

    def expert_ranks(self, expert: int, num_experts: int) -> List[int]:
        if self.ep == 1:
            return list(self.ranks)
        return [self.ranks[expert // (num_experts // self.ep)]]


@dataclass
class Block:
    """One separately sharded piece of a (possibly fused) parameter."""
    infer_name: str
    size: int            # extent along the parameter's shard dimension (whole tensor)


@dataclass
class ParamSpec:
    train_name: str
    shape: Tuple[int, ...]                 # whole parameter, fused blocks included
    shard_dim: int                         # -1 replicated, else the tensor-parallel dimension
    blocks: List[Block] = field(default_factory=list)   # empty: one block named infer_name
    infer_name: str = ""
    groups: int = 1                        # the training shard interleaves the blocks per group (query groups of linear_qkv)
    layer: Optional[int] = None            # transformer layer (decides the pipeline stage); None: see ``where``
    where: str = "layer"                   # "first" / "last" stage for embeddings, final norm and output layer
    expert: Optional[int] = None
    infer_fused_name: Optional[str] = None  # set: the inference side gets the blocks concatenated under this name

    def the_blocks(self) -> List[Block]:
        if self.blocks:
            return self.blocks
        size = self.shape[self.shard_dim] if self.shard_dim >= 0 else 0
        return [Block(self.infer_name or self.train_name, size)]


def decoder_specs(num_layers: int, hidden: int, ffn: int, heads: int, kv_heads: int, head_dim: int, vocab: int,
                  num_experts: int = 0, moe_ffn: int = 0, tie_embeddings: bool = False, fuse_for_inference: bool = False,
                  qkv_bias: bool = False, qk_norm: bool = False) -> Tuple[List[ParamSpec], dict]:
    """Parameter table of a Llama / Qwen style decoder in Megatron-core naming on the training side and Hugging Face
    naming on the inference side. With ``num_experts`` the MLP of every layer is a routed mixture (router + experts).
    ``qkv_bias``: the attention projections carry a bias (Qwen2; fused and interleaved per query group like the weight);
    ``qk_norm``: a per-head RMS norm on queries and keys (Qwen3; replicated).
    -> (specs, meta) where meta carries num_layers / num_experts for the layouts."""
    specs: List[ParamSpec] = []
    q, kv = heads * head_dim, kv_heads * head_dim
    specs.append(ParamSpec("embedding.word_embeddings.weight", (vocab, hidden), 0, infer_name="model.embed_tokens.weight", where="first"))
    for i in range(num_layers):
        t, h = f"decoder.layers.{i}.", f"model.layers.{i}."
        specs.append(ParamSpec(t + "self_attention.linear_qkv.layer_norm_weight", (hidden,), -1, infer_name=h + "input_layernorm.weight", layer=i))
        specs.append(ParamSpec(t + "self_attention.linear_qkv.weight", (q + 2 * kv, hidden), 0, layer=i, groups=kv_heads,
                               blocks=[Block(h + "self_attn.q_proj.weight", q), Block(h + "self_attn.k_proj.weight", kv),
                                       Block(h + "self_attn.v_proj.weight", kv)],
                               infer_fused_name=h + "self_attn.qkv_proj.weight" if fuse_for_inference else None))
        if qkv_bias:
            specs.append(ParamSpec(t + "self_attention.linear_qkv.bias", (q + 2 * kv,), 0, layer=i, groups=kv_heads,
                                   blocks=[Block(h + "self_attn.q_proj.bias", q), Block(h + "self_attn.k_proj.bias", kv),
                                           Block(h + "self_attn.v_proj.bias", kv)],
                                   infer_fused_name=h + "self_attn.qkv_proj.bias" if fuse_for_inference else None))
        if qk_norm:
            specs.append(ParamSpec(t + "self_attention.q_layernorm.weight", (head_dim,), -1, infer_name=h + "self_attn.q_norm.weight", layer=i))
            specs.append(ParamSpec(t + "self_attention.k_layernorm.weight", (head_dim,), -1, infer_name=h + "self_attn.k_norm.weight", layer=i))
        specs.append(ParamSpec(t + "self_attention.linear_proj.weight", (hidden, q), 1, infer_name=h + "self_attn.o_proj.weight", layer=i))
        if num_experts == 0:
            specs.append(ParamSpec(t + "mlp.linear_fc1.layer_norm_weight", (hidden,), -1, infer_name=h + "post_attention_layernorm.weight", layer=i))
            specs.append(ParamSpec(t + "mlp.linear_fc1.weight", (2 * ffn, hidden), 0, layer=i,
                                   blocks=[Block(h + "mlp.gate_proj.weight", ffn), Block(h + "mlp.up_proj.weight", ffn)],
                                   infer_fused_name=h + "mlp.gate_up_proj.weight" if fuse_for_inference else None))
            specs.append(ParamSpec(t + "mlp.linear_fc2.weight", (hidden, ffn), 1, infer_name=h + "mlp.down_proj.weight", layer=i))
        else:
            specs.append(ParamSpec(t + "pre_mlp_layernorm.weight", (hidden,), -1, infer_name=h + "post_attention_layernorm.weight", layer=i))
            specs.append(ParamSpec(t + "mlp.router.weight", (num_experts, hidden), -1, infer_name=h + "mlp.gate.weight", layer=i))
            for e in range(num_experts):
                te, he = t + f"mlp.experts.local_experts.{e}.", h + f"mlp.experts.{e}."
                specs.append(ParamSpec(te + "linear_fc1.weight", (2 * moe_ffn, hidden), 0, layer=i, expert=e,
                                       blocks=[Block(he + "gate_proj.weight", moe_ffn), Block(he + "up_proj.weight", moe_ffn)],
                                       infer_fused_name=he + "gate_up_proj.weight" if fuse_for_inference else None))
                specs.append(ParamSpec(te + "linear_fc2.weight", (hidden, moe_ffn), 1, infer_name=he + "down_proj.weight", layer=i, expert=e))
    specs.append(ParamSpec("decoder.final_layernorm.weight", (hidden,), -1, infer_name="model.norm.weight", where="last"))
    if not tie_embeddings:
        specs.append(ParamSpec("output_layer.weight", (vocab, hidden), 0, infer_name="lm_head.weight", where="last"))
    return specs, {"num_layers": num_layers, "num_experts": num_experts}


def train_shard_of(spec: ParamSpec, full_blocks: Sequence[torch.Tensor], mesh_size: int, index: int) -> torch.Tensor:
    """The shard of ``spec`` that tensor-parallel rank ``index`` of ``mesh_size`` holds in training, from the whole blocks
    (used to build test fixtures and to document the training layout: per group, every block's slice, concatenated)."""
    if spec.shard_dim < 0:
        return full_blocks[0].clone()
    d = spec.shard_dim
    if len(full_blocks) == 1:
        b0, b1 = shard_bounds(full_blocks[0].shape[d], mesh_size, index)
        return full_blocks[0].narrow(d, b0, b1 - b0).contiguous()
    G = spec.groups
    parts = []
    g0, g1 = shard_bounds(G, mesh_size, index) if G > 1 else (0, 1)
    for g in range(g0, g1):
        for blk in full_blocks:
            if G > 1:
                per = blk.shape[d] // G
                parts.append(blk.narrow(d, g * per, per))
            else:
                b0, b1 = shard_bounds(blk.shape[d], mesh_size, index)
                parts.append(blk.narrow(d, b0, b1 - b0))
    return torch.cat(parts, dim=d).contiguous()


class TrainToInferResharder:
    def __init__(self, specs: Sequence[ParamSpec], train: TrainLayout, infer: InferLayout, rank: int, executor, meta: Optional[dict] = None,
                 backend: str = "gloo", bucket_bytes: int = 256 << 20):
        self.specs, self.train, self.infer, self.rank, self.executor = list(specs), train, infer, rank, executor
        meta = meta or {}
        self.num_layers = meta.get("num_layers") or (1 + max((s.layer for s in specs if s.layer is not None), default=0))
        self.num_experts = meta.get("num_experts") or (1 + max((s.expert for s in specs if s.expert is not None), default=-1))
        self.backend = backend
        self.bucket_bytes = bucket_bytes
        self.moved_bytes = 0        # bytes this rank sent or received through the executor (for reports)

    # ------------------------------------------------------------------ layout queries
    def train_mesh(self, spec: ParamSpec) -> List[int]:
        if spec.where == "first" and spec.layer is None:
            stage = 0
        elif spec.where == "last" and spec.layer is None:
            stage = self.train.pp - 1
        else:
            stage = self.train.stage_of_layer(spec.layer, self.num_layers)
        if spec.expert is not None:
            return self.train.expert_ranks(stage, spec.expert, self.num_experts)
        return self.train.stage_ranks(stage)

    def infer_mesh(self, spec: ParamSpec) -> List[int]:
        if spec.expert is not None:
            return self.infer.expert_ranks(spec.expert, self.num_experts)
        return list(self.infer.ranks)

    def holds(self, spec: ParamSpec) -> bool:
        return self.rank in self.train_mesh(spec)

    # ------------------------------------------------------------------ one parameter -> block tensors
    def _local_blocks(self, spec: ParamSpec, local: torch.Tensor, mesh: List[int]) -> List[torch.Tensor]:
        """Splits this rank's training shard into the shards of the separately planned blocks."""
        blocks = spec.the_blocks()
        if len(blocks) == 1:
            return [local]
        d, n, i = spec.shard_dim, len(mesh), mesh.index(self.rank)
        if spec.groups > 1:
            if spec.groups % n != 0:
                raise ValueError(f"{spec.train_name}: {spec.groups} groups do not divide over {n} ranks")
            gl = spec.groups // n
            per = [b.size // spec.groups for b in blocks]
            # [groups_local, sum(per), ...] along d -> one gathered tensor per block
            shp = list(local.shape)
            view = local.reshape(shp[:d] + [gl, sum(per)] + shp[d + 1:])
            out, off = [], 0
            for p in per:
                piece = view.narrow(d + 1, off, p)
                out.append(piece.reshape(shp[:d] + [gl * p] + shp[d + 1:]).contiguous())
                off += p
            return out
        out, off = [], 0
        for b in blocks:
            b0, b1 = shard_bounds(b.size, n, i)
            out.append(local.narrow(d, off, b1 - b0).contiguous())
            off += b1 - b0
        return out

    def _plan_bucket(self, bucket: Sequence[ParamSpec], state: Dict[str, torch.Tensor]):
        pts, meshes, owners = [], [], []
        for spec in bucket:
            tmesh, imesh = self.train_mesh(spec), self.infer_mesh(spec)
            mine = self.rank in tmesh
            local_blocks = None
            if mine:
                if spec.train_name not in state:
                    raise KeyError(f"rank {self.rank} is in the training mesh of {spec.train_name} but its state dict lacks it")
                local_blocks = self._local_blocks(spec, state[spec.train_name], tmesh)
            dtype = self._dtype(spec, state)
            for bi, blk in enumerate(spec.the_blocks()):
                shape = list(spec.shape)
                if spec.shard_dim >= 0:
                    shape[spec.shard_dim] = blk.size
                pts.append(PTensor(local_blocks[bi] if mine else None, dtype, len(shape), tmesh, tuple(shape), spec.shard_dim, rank=self.rank,
                                   backend=self.backend))
                meshes.append(imesh)
                owners.append((spec, blk))
        return pts, meshes, owners

    def _dtype(self, spec: ParamSpec, state: Dict[str, torch.Tensor]) -> torch.dtype:
        if spec.train_name in state:
            return state[spec.train_name].dtype
        return self._default_dtype

    # ------------------------------------------------------------------ the generator
    def per_tensor(self, state: Dict[str, torch.Tensor], dtype: Optional[torch.dtype] = None) -> Iterator[Tuple[str, torch.Tensor]]:
        """Moves every parameter; yields (inference name, this rank's inference shard) on the inference ranks. ``dtype``:
        the parameters' dtype for ranks that hold none of them (defaults to the dtype of any local tensor, else bf16).
        Every rank of both layouts must run the generator to its end."""
        self._default_dtype = dtype or next((t.dtype for t in state.values()), torch.bfloat16)
        for bucket in self._buckets():
            pts, meshes, owners = self._plan_bucket(bucket, state)
            ps = PTensorSet(pts)
            ps.transfer_map(meshes)
            tasks = ps.get_transfer_list()
            self.moved_bytes += sum(self._task_bytes(t) for t in tasks)
            self.executor.execute(tasks)
            self.executor.wait()
            got = ps.collect_tensor()
            k = 0
            for spec in bucket:
                n = len(spec.the_blocks())
                parts = got[k:k + n]
                names = [b.infer_name for b in spec.the_blocks()]
                k += n
                if parts[0] is None:
                    continue
                if spec.infer_fused_name and n > 1:
                    yield spec.infer_fused_name, torch.cat(parts, dim=spec.shard_dim)
                else:
                    for nm, p in zip(names, parts):
                        yield nm, p

    @staticmethod
    def _task_bytes(t) -> int:
        if getattr(t, "size", 0):
            return int(t.size)
        return int(t.numel or 0) * (t.buffer.element_size() if t.buffer is not None else 0)

    def _buckets(self) -> List[List[ParamSpec]]:
        out, cur, size = [], [], 0
        for s in self.specs:
            n = 1
            for x in s.shape:
                n *= x
            nbytes = n * 2
            if cur and size + nbytes > self.bucket_bytes:
                out.append(cur)
                cur, size = [], 0
            cur.append(s)
            size += nbytes
        if cur:
            out.append(cur)
        return out

    def expected_infer_shard(self, spec: ParamSpec, block_index: int, full_block: torch.Tensor, rank: int) -> Optional[torch.Tensor]:
        """What ``rank`` must end up with for one block, from the whole block (for checks)."""
        mesh = self.infer_mesh(spec)
        if rank not in mesh:
            return None
        if spec.shard_dim < 0:
            return full_block
        b0, b1 = shard_bounds(full_block.shape[spec.shard_dim], len(mesh), mesh.index(rank))
        return full_block.narrow(spec.shard_dim, b0, b1 - b0)
