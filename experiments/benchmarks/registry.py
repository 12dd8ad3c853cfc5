"""The measurement grids, declared as data.

Every experiment has registry metadata (name, description, category, whether it takes seeds, output files) and a
``cells`` list: each cell is the keyword set of one ``common.run_config`` / ``common.gradient_fidelity`` call.  The
runner in ``grids.py`` executes the cells; the dry-run planner records them.  The 51 experiment names and what each
one measures follow experiments/benchmarks/registry.py:3-417 of the reference project.
"""

from __future__ import annotations

R8 = dict(rank=8, residual_budget=0.005, residual_bits=8, surface="mlp", min_features=256, chunk_rows=512)
TURBO = dict(R8, turbo_after_step=2)
LOWRANK = dict(R8, residual_budget=0.0, residual_mode="none")
GPT2M = dict(model_id="gpt2-medium", bs=8, seq=1024)
GPT2L = dict(model_id="gpt2-large", bs=4, seq=1024)
PYTHIA = dict(model_id="pythia-1.4b", bs=4, seq=1024)
LLAMA1B = dict(model_id="llama-3.2-1b", bs=2, seq=1024)
QWEN15 = dict(model_id="qwen2.5-1.5b", bs=2, seq=1024)
LLAMA8B = dict(model_id="llama-3.1-8b", bs=1, seq=4096, model_dtype="bfloat16")
QWEN7B = dict(model_id="qwen2.5-7b", bs=1, seq=4096, model_dtype="bfloat16")
SWIGLU = dict(R8, min_features=256)


def _arms(base, arms, **common):
    return [dict(base, method=name, **common, **kw) for name, kw in arms]


STANDARD_ARMS = [("baseline", {}), ("stacr_r8", dict(stacr_cfg=R8)), ("turbo_fast", dict(stacr_cfg=TURBO))]
CKPT_ARMS = [("ckpt_k1", dict(ckpt_every=1)), ("ckpt_k2", dict(ckpt_every=2)), ("ckpt_k4", dict(ckpt_every=4)),
             ("ckpt_k2_plus_turbo", dict(ckpt_every=2, stacr_cfg=TURBO, complement=2)), ("ckpt_k4_plus_turbo", dict(ckpt_every=4, stacr_cfg=TURBO, complement=4))]


def _meta(name, description, category, standard=True, seeds=True, **more):
    return {"name": name, "module": "grids", "description": description, "category": category, "standard": standard, "seeds": seeds, **more}


EXPERIMENTS = {
    "hardware_runtime": _meta("hardware_runtime", "Runtime and model scale across GPU memory capacities", "systems", output_files=["<STACR_HWTAG>.jsonl"],
                              cells=_arms(GPT2M, STANDARD_ARMS) + _arms(PYTHIA, STANDARD_ARMS) + _arms(QWEN7B, [("baseline", {}), ("stacr_mlp_r8", dict(stacr_cfg=SWIGLU))])),
    "attention_kernels": _meta("attention_kernels", "Eager, SDPA, and FlashAttention at the same saved surface", "systems",
                               cells=[dict(GPT2M, method=f"{a}_{m}", attn_impl=a, **kw) for a in ("eager", "sdpa", "flash_attention_2") for m, kw in STANDARD_ARMS]),
    "basis_comparison": _meta("basis_comparison", "STAC-R, Oja-only, OASIS, PRAC, and random basis controls", "quality",
                              cells=[dict(GPT2M, method=k, comparator=k, stacr_cfg=R8) for k in ("stacr", "lowrank", "oasis", "prac", "untracked")] + _arms(GPT2M, [("baseline", {})])),
    "bert_sst2": _meta("bert_sst2", "BERT classification accuracy with full compression and Turbo-fast", "quality", standard=False,
                       cells=_arms(dict(model_id="bert-base-uncased", bs=32, seq=128, task="sequence_classification"), STANDARD_ARMS)),
    "architecture_breadth": _meta("architecture_breadth", "Nine additional transformer families and checkpoint composition", "deployment",
                                  output_files=["x9_breadth.jsonl", "x9_breadth_smoke.jsonl"],
                                  cells=[dict(model_id=m, bs=2, seq=512, method=a, **kw) for m in ("gpt2", "gpt2-large", "pythia-410m", "pythia-1b", "pythia-2.8b", "llama-3.2-1b", "llama-3.2-3b", "qwen2.5-1.5b", "bert-large-uncased")
                                         for a, kw in STANDARD_ARMS + [("ckpt_k2_plus_turbo", dict(ckpt_every=2, stacr_cfg=TURBO, complement=2))]]),
    "budget_throughput": _meta("budget_throughput", "Batch and sequence throughput under a fixed memory budget", "deployment", seeds=False,
                               cells=[dict(GPT2L, method=a, bs=b, **kw) for b in (4, 8, 12, 16) for a, kw in (("baseline", {}), ("hybrid_r8", dict(stacr_cfg=R8)), ("lowrank_r30", dict(stacr_cfg=dict(LOWRANK, rank=30))))]),
    "capacity": _meta("capacity", "GPT-2 model and batch feasibility probes", "deployment", seeds=False,
                      cells=[dict(model_id=m, bs=b, seq=1024, steps=6, measure_from=2, method=a, **kw) for m in ("gpt2-medium", "gpt2-large", "gpt2-xl") for b in (8, 16, 24) for a, kw in (("baseline", {}), ("turbo_fast", dict(stacr_cfg=TURBO)))]),
    "capacity_search": _meta("capacity_search", "Ascending batch search to the first allocation failure", "deployment", seeds=False,
                             cells=[dict(GPT2M, method=a, bs=b, steps=4, measure_from=1, probe="ascending", **kw) for a, kw in (("baseline", {}), ("turbo_fast", dict(stacr_cfg=TURBO))) for b in range(8, 65, 8)]),
    "checkpoint_surface": _meta("checkpoint_surface", "Saved-surface depletion as checkpoint density increases", "mechanism", seeds=False,
                                cells=[dict(GPT2M, method=f"ckpt_k{k}_{a}", ckpt_every=k, **kw) for k in (0, 8, 4, 2, 1) for a, kw in (("plain", {}), ("turbo", dict(stacr_cfg=TURBO, complement=k or None)))]),
    "basis_fidelity": _meta("basis_fidelity", "Dropout-pinned gradient fidelity of basis controls", "fidelity", seeds=False,
                            cells=[dict(kind="fidelity", model_id="gpt2-medium", comparator=k, stacr_cfg=R8, steps=12) for k in ("stacr", "lowrank", "oasis", "prac", "untracked")]),
    "composed_frontier": _meta("composed_frontier", "Checkpoint density, Turbo-fast, full residual, and quality frontier", "deployment",
                               cells=_arms(GPT2M, STANDARD_ARMS + CKPT_ARMS + [("ckpt_k2_plus_full", dict(ckpt_every=2, stacr_cfg=R8, complement=2))])),
    "composition_law": _meta("composition_law", "Additive memory prediction across six basis/compression choices", "mechanism",
                             cells=[dict(GPT2M, method=f"{c}_k{k}", comparator=c, stacr_cfg=R8, ckpt_every=k, complement=k or None) for c in ("stacr", "lowrank", "oasis", "prac", "untracked", "turbo") for k in (0, 2, 4)]),
    "freeze_offload_controls": _meta("freeze_offload_controls", "Frozen MLP and CPU activation offload controls", "mechanism",
                                     cells=_arms(GPT2M, [("baseline", {}), ("freeze_mlp", dict(freeze_mlp=True)), ("offload_all", dict(offload_every=1)), ("offload_half", dict(offload_every=2)), ("turbo_fast", dict(stacr_cfg=TURBO))])),
    "distributed_data": _meta("distributed_data", "DDP per-rank peak and checkpoint composition; launch with torchrun", "distributed", standard=False, module="distributed_data",
                              cells=_arms(dict(model_id="gpt2-medium", bs=4, seq=1024, steps=120, measure_from=20), STANDARD_ARMS + [("ckpt_k4", dict(ckpt_every=4)), ("ckpt_k4_plus_turbo", dict(ckpt_every=4, stacr_cfg=TURBO, complement=4)), ("ckpt_k2", dict(ckpt_every=2)), ("ckpt_k2_plus_turbo", dict(ckpt_every=2, stacr_cfg=TURBO, complement=2))])),
    "allocator_stability": _meta("allocator_stability", "Allocated, reserved, and NVML memory over 600 steps", "systems", standard=False, seeds=False,
                                 cells=_arms(dict(GPT2M, steps=600, measure_from=0, trace_memory=True), STANDARD_ARMS)),
    "equal_budget_frontier": _meta("equal_budget_frontier", "Sparse checkpoint schedules bracketing equal memory and time", "deployment",
                                   cells=[dict(GPT2M, method=f"ckpt_k{k}", ckpt_every=k) for k in (3, 4, 6, 8, 12)] + _arms(GPT2M, STANDARD_ARMS)),
    "precision_corpus": _meta("precision_corpus", "FP32 model controls and OpenWebText corpus comparison", "quality",
                              cells=[dict(GPT2M, method=f"{a}_{d}_{amp}", dataset=d, amp=amp == "bf16", **kw) for d in ("wikitext", "openwebtext") for amp in ("fp32", "bf16") for a, kw in STANDARD_ARMS]),
    "fidelity_horizon": _meta("fidelity_horizon", "Basis adaptation over 6 to 240 pinned-gradient steps", "fidelity", seeds=False,
                              cells=[dict(kind="fidelity", model_id="gpt2-medium", stacr_cfg=R8, steps=s) for s in (6, 12, 30, 60, 120, 240)]),
    "single_model_fidelity": _meta("single_model_fidelity", "Exact and compressed gradients using one model in memory", "fidelity", standard=False, seeds=False,
                                   cells=[dict(kind="fidelity", model_id=m, stacr_cfg=R8, steps=6, single_model=True) for m in ("gpt2-medium", "pythia-1.4b")]),
    "checkpoint_frontier": _meta("checkpoint_frontier", "Full/selective checkpointing and disjoint/overlapping compression", "deployment",
                                 cells=_arms(GPT2M, CKPT_ARMS + [("ckpt_k2_overlap_turbo", dict(ckpt_every=2, stacr_cfg=TURBO)), ("ckpt_k1_overlap_turbo", dict(ckpt_every=1, stacr_cfg=TURBO))])),
    "distributed_sharding": _meta("distributed_sharding", "FSDP2 per-rank memory up to 14B; launch with torchrun", "distributed", standard=False, module="distributed_sharding",
                                  cells=[dict(model_id=m, bs=2, seq=1024, method=a, **kw) for m in ("qwen2.5-1.5b", "llama-3.2-3b", "qwen2.5-7b", "qwen2.5-14b") for a, kw in (("baseline", {}), ("turbo_fast", dict(stacr_cfg=dict(SWIGLU, turbo_after_step=2))))]),
    "training_horizon": _meta("training_horizon", "Long-horizon quality on WikiText and OpenWebText", "quality",
                              cells=[dict(GPT2M, method=a, dataset=d, steps=s, measure_from=20, **kw) for d in ("wikitext", "openwebtext") for s in (400, 1000) for a, kw in STANDARD_ARMS]),
    "composition_architectures": _meta("composition_architectures", "Composition-law validation on Pythia and Qwen", "mechanism",
                                       cells=[dict(base, method=f"{a}", **kw) for base in (PYTHIA, QWEN15) for a, kw in STANDARD_ARMS + CKPT_ARMS]),
    "training_2000": _meta("training_2000", "Seven GPT-2 Medium training arms at 2000 steps", "quality",
                           cells=_arms(dict(GPT2M, steps=2000, measure_from=20), STANDARD_ARMS + [("ckpt_k1", dict(ckpt_every=1)), ("lowrank_r8", dict(stacr_cfg=LOWRANK)), ("stacr_r32", dict(stacr_cfg=dict(R8, rank=32))), ("turbo_at_50", dict(stacr_cfg=dict(R8, turbo_after_step=50)))])),
    "training_2000_composition": _meta("training_2000_composition", "Disjoint full-residual composition at 2000 steps", "quality",
                                       cells=_arms(dict(GPT2M, steps=2000, measure_from=20), [("ckpt_k2_plus_full", dict(ckpt_every=2, stacr_cfg=R8, complement=2)), ("ckpt_k4_plus_full", dict(ckpt_every=4, stacr_cfg=R8, complement=4))])),
    "lora": _meta("lora", "LoRA and full training memory; BERT labels are synthetic", "deployment", standard=False,
                  cells=[dict(model_id=m, bs=8, seq=512, method=f"{t}_{a}", lora=t == "lora", **kw) for m in ("gpt2-medium", "bert-base-uncased") for t in ("full", "lora") for a, kw in STANDARD_ARMS]),
    "modern_architectures": _meta("modern_architectures", "Qwen3 and 3B-tier model surfaces and batch sizes", "deployment", seeds=False,
                                  cells=[dict(model_id=m, bs=b, seq=1024, method=a, **kw) for m in ("qwen2.5-1.5b", "llama-3.2-3b") for b in (1, 2, 4) for a, kw in (("baseline", {}), ("turbo_fast", dict(stacr_cfg=dict(SWIGLU, turbo_after_step=2))))]),
    "modern_composition": _meta("modern_composition", "Checkpoint density and Turbo-fast on modern decoder MLPs", "deployment",
                                cells=[dict(base, method=a, **kw) for base in (LLAMA1B, QWEN15) for a, kw in CKPT_ARMS + [("baseline", {})]]),
    "modern_precision": _meta("modern_precision", "Precision controls and 600-step modern-model quality", "quality",
                              cells=[dict(base, method=f"{a}_{p}", steps=600, model_dtype=p, **kw) for base in (LLAMA1B, QWEN15) for p in ("float32", "bfloat16") for a, kw in STANDARD_ARMS]),
    "runtime_breakdown": _meta("runtime_breakdown", "Refresh interval, frozen basis, and quantized residual overhead", "systems",
                               cells=_arms(GPT2M, STANDARD_ARMS + [(f"update_every_{k}", dict(stacr_cfg=dict(R8, update_interval=k))) for k in (2, 4, 10, 50)] + [("frozen_basis", dict(stacr_cfg=dict(R8, freeze_after_warmup=True, warmup_steps=2))), ("residual_fp", dict(stacr_cfg=dict(R8, residual_bits=0))), ("residual_int4", dict(stacr_cfg=dict(R8, residual_bits=4)))])),
    "peak_anatomy": _meta("peak_anatomy", "Training-phase allocation and chunked cross-entropy controls", "mechanism", standard=False, seeds=False,
                          cells=_arms(dict(GPT2M, phase_profile=True), STANDARD_ARMS + [("chunked_ce", dict(model_overrides=dict(loss_chunk=2048)))])),
    "principal_random_rank": _meta("principal_random_rank", "PRAC at recommended rank versus STAC-R at matched rank", "fidelity",
                                   cells=[dict(kind="fidelity", model_id="gpt2-medium", comparator=c, stacr_cfg=dict(R8, rank=r), steps=12) for c in ("prac", "stacr") for r in (8, 307)]),
    "pythia": _meta("pythia", "Pythia-1.4B baseline, checkpoint, full residual, and Turbo-fast", "quality", cells=_arms(PYTHIA, STANDARD_ARMS + [("ckpt_k1", dict(ckpt_every=1))])),
    "qlora": _meta("qlora", "NF4 QLoRA memory and supported composition; synthetic BERT labels", "deployment", standard=False,
                   cells=[dict(model_id=m, bs=8, seq=512, method=f"qlora_{a}", qlora=True, **kw) for m in ("gpt2-large", "bert-base-uncased") for a, kw in STANDARD_ARMS]),
    "rate_distortion": _meta("rate_distortion", "Stored-byte and gradient-error frontier over rank and basis", "fidelity", seeds=False,
                             cells=[dict(kind="fidelity", model_id="gpt2-medium", comparator=c, stacr_cfg=dict(R8, rank=r, residual_budget=b), steps=6) for c in ("stacr", "untracked") for r in (4, 8, 16, 30, 64, 128) for b in (0.0, 0.005)]),
    "parameter_sweep": _meta("parameter_sweep", "Rank, residual budget, and basis-update operating points", "deployment",
                             cells=[dict(GPT2M, method=f"r{r}_b{b}_u{u}", stacr_cfg=dict(R8, rank=r, residual_budget=b, update_interval=u)) for r in (4, 8, 16, 32) for b in (0.0, 0.0025, 0.005, 0.01) for u in (1, 4)]),
    "residual_budget": _meta("residual_budget", "Residual on/off, 0.5%, and 1% quality-memory-time tradeoffs", "quality",
                             cells=_arms(GPT2M, [("baseline", {})] + [(f"budget_{b}", dict(stacr_cfg=dict(R8, residual_budget=b))) for b in (0.0, 0.005, 0.01)])),
    "residual_selectors": _meta("residual_selectors", "Chunked, global, block-sparse, and sampled residual selection", "systems",
                                cells=_arms(GPT2M, [(m, dict(stacr_cfg=dict(R8, residual_mode=m))) for m in ("chunk_topk", "global_topk", "block_sparse", "sampled", "uniform")])),
    "large_models": _meta("large_models", "7B/8B context lengths, batches, and composed memory frontier", "deployment",
                          cells=[dict(base, method=a, seq=s, **kw) for base in (LLAMA8B, QWEN7B) for s in (2048, 4096) for a, kw in (("baseline", {}), ("turbo_fast", dict(stacr_cfg=dict(SWIGLU, turbo_after_step=2))), ("ckpt_k2_plus_turbo", dict(ckpt_every=2, stacr_cfg=dict(SWIGLU, turbo_after_step=2), complement=2)))]),
    "large_model_fidelity": _meta("large_model_fidelity", "Single-model gradient probes on 7B/8B and Pythia", "fidelity", standard=False, seeds=False,
                                  cells=[dict(kind="fidelity", model_id=m, stacr_cfg=SWIGLU, steps=4, single_model=True) for m in ("llama-3.1-8b", "qwen2.5-7b", "pythia-1.4b")]),
    "sequence_length": _meta("sequence_length", "Context-length and batch capacity on Llama and Qwen", "deployment",
                             cells=[dict(base, method=a, seq=s, bs=1, **kw) for base in (LLAMA1B, QWEN15) for s in (1024, 2048, 4096, 8192, 16384) for a, kw in (("baseline", {}), ("turbo_fast", dict(stacr_cfg=dict(SWIGLU, turbo_after_step=2))))]),
    "surface_expansion": _meta("surface_expansion", "MLP, attention, and all-linear compression on GPT-2", "deployment",
                               cells=_arms(GPT2L, [("baseline", {})] + [(f"surface_{s.replace('+', '_')}", dict(stacr_cfg=dict(R8, surface=s))) for s in ("mlp", "attention", "mlp+attention", "all")])),
    "modern_surfaces": _meta("modern_surfaces", "Modern-model surface expansion and its quality cost", "deployment",
                             cells=[dict(base, method=f"surface_{s.replace('+', '_')}", stacr_cfg=dict(SWIGLU, surface=s)) for base in (LLAMA1B, QWEN15) for s in ("mlp", "mlp+attention", "all")]),
    "swiglu_surfaces": _meta("swiglu_surfaces", "SwiGLU rank, token shape, and down-projection surface sweep", "mechanism", seeds=False,
                             cells=[dict(LLAMA1B, method=f"r{r}_{t}", bs=b, seq=s, stacr_cfg=dict(SWIGLU, rank=r, target_pattern=p)) for r in (8, 32) for (b, s) in ((2, 1024), (8, 256)) for t, p in (("all_mlp", None), ("down_only", "down_proj"))]),
    "swiglu_precision": _meta("swiglu_precision", "SwiGLU precision and optimizer allocation controls", "mechanism", seeds=False,
                              cells=[dict(LLAMA1B, method=f"{a}_{p}_{o}", model_dtype=p, eight_bit=o == "adamw8bit", **kw) for p in ("float32", "bfloat16") for o in ("adamw", "adamw8bit") for a, kw in (("baseline", {}), ("turbo_fast", dict(stacr_cfg=dict(SWIGLU, turbo_after_step=2))))]),
    "swiglu_shape_fidelity": _meta("swiglu_shape_fidelity", "Pinned gradient fidelity at two-example 1024-token shapes", "fidelity", seeds=False,
                                   cells=[dict(kind="fidelity", model_id=m, stacr_cfg=SWIGLU, bs=2, seq=1024, steps=6) for m in ("llama-3.2-1b", "qwen2.5-1.5b")]),
    "swiglu_fidelity": _meta("swiglu_fidelity", "Rank and residual fidelity on three modern decoder families", "fidelity", seeds=False,
                             cells=[dict(kind="fidelity", model_id=m, stacr_cfg=dict(SWIGLU, rank=r, residual_budget=b), steps=6) for m in ("llama-3.2-1b", "qwen2.5-1.5b", "llama-3.2-3b") for r in (8, 32) for b in (0.0, 0.005)]),
    "swiglu_composition": _meta("swiglu_composition", "Same-block versus disjoint checkpoint composition on SwiGLU", "deployment", seeds=False,
                                cells=[dict(LLAMA1B, method=a, **kw) for a, kw in (("ckpt_k2", dict(ckpt_every=2)), ("ckpt_k2_same_block_turbo", dict(ckpt_every=2, stacr_cfg=dict(SWIGLU, turbo_after_step=2))), ("ckpt_k2_disjoint_turbo", dict(ckpt_every=2, stacr_cfg=dict(SWIGLU, turbo_after_step=2), complement=2)))]),
    "basis_storage": _meta("basis_storage", "Allocation-only duplicated-basis and residual-storage controls", "mechanism", seeds=False,
                           cells=[dict(GPT2M, method=f"basis_{d}", stacr_cfg=dict(R8, basis_dtype=d)) for d in ("float32", "bfloat16")] + [dict(GPT2M, method=f"residual_bits_{b}", stacr_cfg=dict(R8, residual_bits=b)) for b in (0, 4, 8)]
                           + [dict(GPT2M, method=f"fat_{n}", comparator="fat", stacr_cfg=dict(R8, basis_per_call=b, fat_residual=f)) for n, b, f in (("basis_per_call", True, False), ("residual", False, True), ("both", True, True))]),
    "subtrack_composition": _meta("subtrack_composition", "Upstream SubTrack++ BERT/SST-2 and adaptive STAC-R composition", "comparators", standard=False,
                                  cells=[dict(model_id="bert-base-uncased", bs=32, seq=128, task="sequence_classification", method=m, optimizer=o, **kw) for m, o, kw in (("subtrack", "subtrack", {}), ("subtrack_stacr", "subtrack", dict(stacr_cfg=R8, engine="adaptive")), ("adamw", "adamw", {}))]),
    "instant_comparison": _meta("instant_comparison", "INSTANT SST-2, MRPC, and GPT-2 protocols with calibration", "comparators", standard=False,
                                cells=[dict(model_id=m, bs=16, seq=128, method=f"{t}_{a}", task=t, **kw) for m, t in (("bert-base-uncased", "sst2"), ("bert-base-uncased", "mrpc"), ("gpt2", "lm")) for a, kw in (("baseline", {}), ("stacr_r8", dict(stacr_cfg=R8)), ("instant_style_lowrank", dict(stacr_cfg=LOWRANK)))]),
}

assert len(EXPERIMENTS) == 51
