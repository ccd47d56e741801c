"""Communication volume model: how many collectives one rank issues per optimizer step and how
many bytes it sends, predicted from the configuration alone.

    python -m shardtrain_b200.utils.comm_volume --config configs/qwen25_1p5b_b200.yaml --strategy F2T2/SP

Two wire formats are modelled:

* `reference` - what the reference runtime moves (FP32 parameter all-gather and gradient
  reduce-scatter through NCCL, a TP all-reduce for replicated parameters, sequence-parallel
  activations in the compute dtype with FP32 input gradients), with the ideal-ring send model its
  own study uses (`experiments/fsdp_interview/cases/q06_comm_volume.py:13-24`,
  `reports/fsdp_interview_sections/04_communication_volume.md:66-92`): an all-gather or
  reduce-scatter over n ranks sends (n-1)/n of the full payload, an all-reduce twice that.
* `peer` - what this package's sm_100a kernels move: matrices are pulled from the owners' bf16
  shadow shards (vectors in FP32), gradients are pulled in FP32 over the whole mesh so the
  replicated parameters need no extra all-reduce, sequence-parallel traffic is unchanged.  A pull
  over n ranks brings in (n-1)/n of the payload, so the same factor applies to bytes received.

The unit plan is the runtime's: the (tied) embedding, every decoder layer, the final norm and,
for untied models, the head.  Per micro-step every unit is gathered for the forward; for the
backward every unit that was resharded is gathered again (not the last unit, and not a tied
embedding, which stays materialised from the lookup to the end of the backward).
"""

from __future__ import annotations

import argparse
import json
from dataclasses import dataclass


@dataclass(frozen=True)
class Unit:
    name: str
    split: int          # elements divided by T (column / row parallel matrices and biases)
    replicated: int     # elements every TP rank holds in full (norms, embedding, head)
    regathered: bool    # gathered a second time for the backward


def qwen_units(m, tp: int) -> list[Unit]:
    """TP-local element counts of every unit of a Qwen2 model (`m`: the model section)."""
    h, inter, heads = m["hidden_size"], m["mlp_hidden_size"], m["num_heads"]
    kv = m.get("num_key_value_heads", heads) * (h // heads)
    layer_split = (h * h + h) + 2 * (kv * h + kv) + h * h + 3 * inter * h     # q,k,v (+bias), o, mlp
    layer = Unit("layer", layer_split // tp, 2 * h, True)
    tied = m.get("tie_word_embeddings", True)
    table = m["vocab_size"] * h
    units = [Unit("embedding", 0, table, not tied)]
    units += [layer] * m["layers"]
    if tied:
        units.append(Unit("final_norm", 0, h, False))
    else:
        units.append(Unit("final_norm", 0, h, True))
        units.append(Unit("head", 0, table, False))
    return units


def qwen_parameters(m, tp: int) -> list[tuple[int, str, int, bool]]:
    """(unit index, name, TP-local element count, replicated over TP) of every parameter, in the
    runtime's unit order."""
    h, inter, heads = m["hidden_size"], m["mlp_hidden_size"], m["num_heads"]
    kv = m.get("num_key_value_heads", heads) * (h // heads)
    table = m["vocab_size"] * h
    rows = [(0, "embed_tokens.weight", table, True)]
    for layer in range(m["layers"]):
        unit = layer + 1
        rows += [(unit, "q_proj.weight", h * h // tp, False), (unit, "q_proj.bias", h // tp, False),
                 (unit, "k_proj.weight", kv * h // tp, False), (unit, "k_proj.bias", kv // tp, False),
                 (unit, "v_proj.weight", kv * h // tp, False), (unit, "v_proj.bias", kv // tp, False),
                 (unit, "o_proj.weight", h * h // tp, False),
                 (unit, "gate_proj.weight", inter * h // tp, False),
                 (unit, "up_proj.weight", inter * h // tp, False),
                 (unit, "down_proj.weight", inter * h // tp, False),
                 (unit, "input_layernorm.weight", h, True),
                 (unit, "post_attention_layernorm.weight", h, True)]
    rows.append((m["layers"] + 1, "norm.weight", h, True))
    if not m.get("tie_word_embeddings", True):
        rows.append((m["layers"] + 2, "lm_head.weight", table, True))
    return rows


def microstep_payload(model: dict, *, fsdp: int, tp: int, sp: bool, local_batch: int) -> dict:
    """What the collectives of ONE micro-step carry on the library-collective path, in elements
    (shards are padded to ceil(n / F), so a gathered parameter is F * ceil(n / F) elements):

    * `fsdp_ag`: gathers issued and the elements they deliver (all units for the forward, the
      resharded ones again for the backward);
    * `fsdp_rs`: elements entering the gradient reductions (every parameter once); the number of
      reductions lies between one per unit and one per bucket (asynchronous reduction puts a
      unit's norm weights in a bucket of their own);
    * `sp_ag` / `sp_rs`: six gathers and four reduce-scatters of a full [batch, sequence, hidden]
      activation per layer;
    * `tp_replicated_allreduce`: one all-reduce per TP-replicated parameter (each norm weight,
      the embedding, an untied head), over its FSDP shard.
    """
    params = qwen_parameters(model, tp)
    tied = model.get("tie_word_embeddings", True)
    last_unit = max(unit for unit, *_ in params)
    padded = lambda n: fsdp * -(-n // fsdp)          # noqa: E731
    regathered = {unit for unit, *_ in params
                  if unit != last_unit and not (tied and unit == 0)}
    units = {unit for unit, *_ in params}
    out = {"fsdp_ag": {"count": len(units) + len(regathered),
                       "elements": sum(padded(n) * (2 if unit in regathered else 1)
                                       for unit, _, n, _ in params)},
           "fsdp_rs": {"count_min": len(units),
                       "count_max": len({(unit, rep) for unit, _, _, rep in params}),
                       "elements": sum(padded(n) for _, _, n, _ in params)}}
    if tp > 1:
        shards = [-(-n // fsdp) for _, _, n, rep in params if rep]
        out["tp_replicated_allreduce"] = {"count": len(shards), "elements": sum(shards)}
        if sp:
            tokens = local_batch * model["seq_len"] * model["hidden_size"]
            out["sp_ag"] = {"count": 6 * model["layers"], "elements": 6 * model["layers"] * tokens}
            out["sp_rs"] = {"count": 4 * model["layers"], "elements": 4 * model["layers"] * tokens}
    return out


def predict(model: dict, *, fsdp: int, tp: int, sp: bool, local_batch: int, accumulation: int,
            compute_bytes: int = 2, wire: str = "reference") -> dict:
    """Counts and bytes per rank per optimizer step, by role."""
    if wire not in ("reference", "peer"):
        raise ValueError("wire must be reference or peer")
    units = qwen_units(model, tp)
    A, L, h = accumulation, model["layers"], model["hidden_size"]
    ring_f, ring_t = (fsdp - 1) / fsdp, (tp - 1) / tp

    def gathered_bytes(unit):
        if wire == "peer":        # bf16 shadow for matrices (everything 2-D), FP32 for vectors
            vectors = 2 * h if unit.name == "layer" else (h if unit.name == "final_norm" else 0)
            bias = 0
            if unit.name == "layer":
                heads = model["num_heads"]
                kvw = model.get("num_key_value_heads", heads) * (h // heads)
                bias = (h + 2 * kvw) // tp
            matrices = unit.split + unit.replicated - vectors - bias
            return 2 * matrices + 4 * (vectors + bias)
        return 4 * (unit.split + unit.replicated)

    forward = sum(gathered_bytes(u) for u in units)
    backward = sum(gathered_bytes(u) for u in units if u.regathered)
    gathers = len(units) + sum(u.regathered for u in units)
    grads = sum(4 * (u.split + u.replicated) for u in units)
    # the reference reduces replicated parameters in a bucket of their own when T > 1
    buckets = sum((1 if u.split else 0) + (1 if u.replicated else 0) for u in units) if tp > 1 \
        else len(units)
    roles = {
        "fsdp_param_allgather": {"count": A * gathers, "bytes": A * ring_f * (forward + backward)},
        "fsdp_grad_reduce_scatter": {"count": A * (buckets if wire == "reference" else len(units)),
                                     "bytes": A * ring_f * grads},
    }
    if wire == "peer" and tp > 1:
        # replicated parameters are summed over the whole F x T mesh inside the same kernel
        replicated = sum(4 * u.replicated for u in units)
        world = fsdp * tp
        roles["fsdp_grad_reduce_scatter"]["bytes"] = A * (
            ring_f * (grads - replicated) + (world - 1) / world * replicated)
    if sp and tp > 1:
        tokens = local_batch * model["seq_len"] * h
        x_compute, x32 = compute_bytes * tokens, 4 * tokens
        roles["sp_activation_allgather"] = {"count": 6 * A * L, "bytes": A * L * ring_t * 6 * x_compute}
        roles["sp_activation_reduce_scatter"] = {"count": 4 * A * L,
                                                 "bytes": A * L * ring_t * (2 * x_compute + 2 * x32)}
    if wire == "reference" and tp > 1:
        norms = 2 * L + 1
        roles["tp_norm_grad_allreduce"] = {"count": A * norms, "bytes": A * norms * 2 * ring_t * 4 * h / fsdp}
        big = [u for u in units if u.name in ("embedding", "head")]
        roles["tp_replicated_grad_allreduce"] = {
            "count": A * len(big), "bytes": A * sum(2 * ring_t * 4 * u.replicated / fsdp for u in big)}
    for role in roles.values():
        role["bytes"] = int(round(role["bytes"]))
    return {"roles": roles, "collectives": sum(r["count"] for r in roles.values()),
            "bytes": sum(r["bytes"] for r in roles.values()), "wire": wire,
            "mesh": {"fsdp": fsdp, "tp": tp, "sp": bool(sp)}}


def main(argv=None) -> int:
    from shardtrain_b200.config import load_config

    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--config", required=True)
    ap.add_argument("--strategy", default=None, help="F{dp}T{tp}[/SP]; default: the config's mesh")
    ap.add_argument("--wire", choices=["reference", "peer", "both"], default="both")
    args = ap.parse_args(argv)
    config = load_config(args.config, ["--parallel.strategy", args.strategy] if args.strategy else [])
    m, p, t = config.model, config.parallel, config.training
    model = dict(hidden_size=m.hidden_size, mlp_hidden_size=m.mlp_hidden_size, num_heads=m.num_heads,
                 num_key_value_heads=m.num_key_value_heads or m.num_heads, layers=m.layers,
                 vocab_size=m.vocab_size, seq_len=m.seq_len, tie_word_embeddings=m.tie_word_embeddings)
    compute = 4 if t.dtype == "fp32" else 2
    for wire in (("reference", "peer") if args.wire == "both" else (args.wire,)):
        print(json.dumps(predict(model, fsdp=p.fsdp_degree, tp=p.tp_degree, sp=p.sp_enabled,
                                 local_batch=t.local_batch_size, accumulation=t.accumulation_steps,
                                 compute_bytes=compute, wire=wire), indent=2))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
