"""Tiered successive-halving sweep: a schedule of tiers, each sampling the plan grid, timing
its sample on the GPUs and seeding the next tier with its winners.

Follows contrib/kittens/test/bench/bench_tier_schedule.py (``TierSpec`` :23-66, axis-value
resolution :79-121, ``apply_tier_overrides`` :124-148) and bench_tier_driver.py
(``run_tier_mode`` :52-275: keep ``min(candidates, max(10 %, 50))`` winners per tier, verify the
final winners, only verified results are emitted).  The policy -- which axes a tier pins,
frees or widens -- belongs to the bench that supplies the schedule; :func:`b200_tier_schedule`
is the one for the B200 plan grid of :func:`aster_b200.bench_search.b200_gemm_grid`.
"""

from __future__ import annotations

import contextlib
import signal
import time
from dataclasses import dataclass, field
from typing import Any, Callable, Optional

from .bench_harness import INIT_DEFAULT, emit_one_result

TIER_KEEP_PCT = 0.10
TIER_KEEP_CAP = 50


def make_constraints(grid) -> tuple:
    """Names of the named filters registered on ``grid``."""
    return tuple(grid.filter_names())


@dataclass(frozen=True)
class TierSpec:
    """One tier.  Axis values resolve per axis, later wins: (1) from the second tier on, the
    union over the previous winners of their own value, its ``neighbor_radius`` ordinal
    neighbours and, for ``free_axes``, every value; (2) ``axis_grid``: explicit values;
    (3) ``fixed_axes``: a pin; (4) the driver's ambient pins.  ``discriminator`` names the axis
    (or axes) whose values are the strata of the sampling; ``constraints`` names the grid's
    filters this tier keeps (anonymous filters always apply); ``per_stratum_diversity`` keeps
    the best config of every stratum before the overall cut."""

    tier_idx: int
    max_configs: int
    random_seed: Optional[int]
    constraints: tuple
    axis_grid: dict = field(default_factory=dict)
    fixed_axes: dict = field(default_factory=dict)
    free_axes: list = field(default_factory=list)
    neighbor_radius: dict = field(default_factory=dict)
    discriminator: Any = None
    per_stratum_diversity: bool = False


def ordinal_neighbors(value, value_list: list, radius: int) -> list:
    """Values within ``radius`` index steps of ``value`` in ``value_list`` (clamped at the ends)."""
    if value not in value_list:
        return [value]
    i = value_list.index(value)
    return value_list[max(0, i - radius): min(len(value_list) - 1, i + radius) + 1]


def tier_axis_overrides(universe: dict, tier: TierSpec, prev_winners: list, ambient_pins: dict) -> dict:
    """``{axis: values}`` for the tier's grid (resolution order of :class:`TierSpec`)."""
    overrides: dict = {}
    if prev_winners:
        union: dict = {}
        for winner in prev_winners:
            base = {k: v for k, v in winner.items() if not k.startswith("_")}
            for k, v in base.items():
                if k in universe:
                    union.setdefault(k, set()).add(v)
            for axis, radius in tier.neighbor_radius.items():
                if axis in base and axis in universe:
                    union.setdefault(axis, set()).update(ordinal_neighbors(base[axis], list(universe[axis]), radius))
            for axis in tier.free_axes:
                if axis in universe:
                    union.setdefault(axis, set()).update(universe[axis])
        for k, vs in union.items():
            overrides[k] = sorted(vs, key=str)
    for k, vals in tier.axis_grid.items():
        overrides[k] = list(vals)
    for k, v in tier.fixed_axes.items():
        overrides[k] = [v]
    for k, v in ambient_pins.items():
        overrides[k] = [v]
    return overrides


def apply_tier_overrides(grid, tier: TierSpec, prev_winners: list, ambient_pins: Optional[dict] = None, *, universe: Optional[dict] = None) -> None:
    """Restrict ``grid`` in place to the tier's axis values and filters.  ``universe`` is the value
    pool of the ordinal-neighbour expansion (normally the first tier's values)."""
    if not universe:
        universe = grid.axis_values()
    overrides = tier_axis_overrides(universe, tier, prev_winners, ambient_pins or {})
    overrides = {k: v for k, v in overrides.items() if k in grid.axis_values()}
    grid.restrict_axes(overrides)
    grid.retain_filters(set(tier.constraints))
    empty = [name for name, vals in grid.axis_values().items() if not vals]
    if empty:
        raise ValueError(f"Tier {tier.tier_idx} left sweep axes with no values {empty!r}; add them to axis_grid or fixed_axes")


def keep_count(n_candidates: int) -> int:
    """Winners a tier hands on: ``min(candidates, max(10 % of them, 50))``."""
    return min(n_candidates, max(int(n_candidates * TIER_KEEP_PCT), TIER_KEEP_CAP))


def select_winners(measured: list, tier: TierSpec) -> list:
    """``measured`` = ``[(axis dict, tflops)]`` -> the winners' axis dicts (``_tflops`` added),
    best first."""
    ranked = sorted(measured, key=lambda m: -m[1])
    keep = keep_count(len(ranked))
    if tier.per_stratum_diversity and tier.discriminator:
        names = tier.discriminator if isinstance(tier.discriminator, tuple) else (tier.discriminator,)
        seen, diverse = set(), []
        for d, tf in ranked:
            key = tuple(d.get(n) for n in names)
            if key not in seen:
                seen.add(key)
                diverse.append((d, tf))
        ranked = diverse + [m for m in ranked if m not in diverse]
    return [dict(d, _tflops=tf) for d, tf in ranked[:keep]]


def _alarm_to_keyboard_interrupt(signum, frame):
    raise KeyboardInterrupt(f"tier time budget exceeded (signal {signum})")


@contextlib.contextmanager
def tier_alarm(budget: Optional[float]):
    """``SIGALRM`` after ``budget`` seconds turns into ``KeyboardInterrupt``, which the sweep
    treats as "stop compiling, drain what is in flight, return what you have"."""
    if not budget or budget <= 0:
        yield
        return
    old = signal.signal(signal.SIGALRM, _alarm_to_keyboard_interrupt)
    signal.alarm(int(budget))
    try:
        yield
    finally:
        signal.alarm(0)
        signal.signal(signal.SIGALRM, old)


def run_tier_mode(*, grid_factory: Callable, tier_schedule: list, sweep_fn: Callable, verify_fn: Optional[Callable] = None,
                  ambient_pins: Optional[dict] = None, bench_label: str = "unknown", results_stream=None, dry_run: bool = False,
                  tier_time_budget: Optional[float] = None, log=print) -> list:
    """Walk ``tier_schedule``.  Each tier: a fresh grid restricted to the tier's values,
    ``generate`` at most ``max_configs`` instances (stratified by the discriminator),
    ``sweep_fn(instances) -> (results, artifact_paths)`` with ``results = [(cfg, stats)]``,
    winners seed the next tier.  After the last tier ``verify_fn(results, artifact_paths) ->
    {labels that passed}`` gates what is written to ``results_stream``: only verified results
    are emitted.  Returns every tier's ``[(cfg, stats)]`` concatenated, fastest first."""
    prev_winners: list = []
    # Value pool of the later tiers' neighbour and free-axis expansion: the unrestricted grid, so
    # that an axis a first tier pins (ring depth, K split) can be opened again by a later one.
    universe: dict = grid_factory().axis_values()
    all_results, all_paths = [], {}
    for tier in tier_schedule:
        grid = grid_factory()
        apply_tier_overrides(grid, tier, prev_winners, ambient_pins, universe=universe)
        if isinstance(tier.discriminator, tuple):
            strat = lambda d, ks=tier.discriminator: tuple(d[k] for k in ks)  # noqa: E731
        elif tier.discriminator:
            strat = lambda d, k=tier.discriminator: d[k]  # noqa: E731
        else:
            strat = None
        instances, cfgs, total = grid.generate(sample_size=tier.max_configs, stratification_key=strat, seed=tier.random_seed or 0)
        log(f"=== Tier {tier.tier_idx}: generated={total}, taken={len(instances)} (cap={tier.max_configs}), discriminator={tier.discriminator!r} ===")
        if dry_run and tier.tier_idx == tier_schedule[0].tier_idx:
            for inst in instances:
                log(f"  {inst.label}")
            return []
        if not instances:
            log(f"Tier {tier.tier_idx}: no candidates; stopping")
            break
        axes_by_label = {inst.label: d for inst, d in zip(instances, cfgs)}
        t0 = time.monotonic()
        with tier_alarm(tier_time_budget):
            try:
                results, paths = sweep_fn(instances)
            except KeyboardInterrupt:
                log(f"Tier {tier.tier_idx}: time budget exceeded before any result was returned")
                results, paths = [], {}
        log(f"Tier {tier.tier_idx}: {len(results)} measured in {time.monotonic() - t0:.1f} s")
        all_results.extend(results)
        all_paths.update(paths)
        measured = [(axes_by_label[cfg.label], stats.p50_tf) for cfg, stats in results if cfg.label in axes_by_label]
        if not measured:
            break
        prev_winners = select_winners(measured, tier)
    all_results.sort(key=lambda r: -r[1].p50_tf)
    if results_stream is not None and all_results:
        verified = verify_fn(all_results, all_paths) if verify_fn is not None else set()
        for cfg, stats in all_results:
            if cfg.label in verified:
                emit_one_result(results_stream, bench_label, cfg, stats)
        log(f"Emitted {len(verified)}/{len(all_results)} verified result(s)")
    return all_results


def b200_tier_schedule(seed: int = 42, cap: int = 24) -> list:
    """Two tiers for the B200 plan grid: first the tile geometry (width x CTA pair) with the
    library's own ring depth and no K split, stratified so that every geometry is tried; then
    ring depth and K split around the winners."""
    constraints = ("tile_not_wider_than_n", "pair_needs_256_rows", "fits_shared_memory", "split_leaves_k_blocks")
    return [
        TierSpec(tier_idx=1, max_configs=cap, random_seed=seed, constraints=constraints, fixed_axes={"stages": 0, "split_k": 0},
                 discriminator=("tile_n", "cta_group"), per_stratum_diversity=True),
        TierSpec(tier_idx=2, max_configs=cap, random_seed=seed + 1, constraints=constraints, free_axes=["stages", "split_k"],
                 neighbor_radius={"tile_n": 1}, discriminator="stages"),
    ]


def main(argv=None) -> int:
    """``python -m aster_b200.bench_tier --mcpu sm_100a --size MxNxK [...]``: the tiered sweep of
    one problem size on the visible GPUs."""
    import argparse
    import sys

    from .bench_search import b200_gemm_grid, parse_mnk
    from .bench_workers import add_sweep_cli_args, bench_perf_sweep_pipelined, require_gpu_or_compile_only, verify_top_configs
    from .multitile_gemm import BENCH_HOOKS

    ap = argparse.ArgumentParser(description=main.__doc__)
    add_sweep_cli_args(ap)
    ap.add_argument("--size", type=parse_mnk, required=True)
    ap.add_argument("--dtype", default="bf16", choices=["f16", "bf16", "e4m3", "e5m2", "i8"])
    ap.add_argument("--out-dtype", default="bf16", choices=["f32", "bf16", "i32"])
    args = ap.parse_args(argv)
    require_gpu_or_compile_only(args)
    m, n, k = args.size
    num_gpus = 0 if args.compile_only else args.num_gpus

    def sweep(instances):
        return bench_perf_sweep_pipelined(instances, BENCH_HOOKS["compile_fn"], BENCH_HOOKS["repro_cmd_fn"], mcpu=args.mcpu,
                                          bench=BENCH_HOOKS["bench_label"], num_gpus=num_gpus, compile_workers=args.compile_workers,
                                          post_compile_filter=None if args.no_reg_filter else BENCH_HOOKS["post_compile_filter"],
                                          init_mode=args.init, iterations=args.iterations, hsaco_dir=args.hsaco_dir)

    def verify(results, paths):
        from .bench_workers import detect_num_gpus

        return verify_top_configs(results, paths, top_n=len(results), num_gpus=args.num_gpus or detect_num_gpus(args.mcpu), init_mode=args.init)

    stream = open(args.results_file, "a") if args.results_file else None
    try:
        ranked = run_tier_mode(grid_factory=lambda: b200_gemm_grid(m, n, k, args.dtype, args.out_dtype),
                               tier_schedule=b200_tier_schedule(args.seed, args.compile_sample or 10 ** 6), sweep_fn=sweep,
                               verify_fn=None if args.compile_only else verify, bench_label=BENCH_HOOKS["bench_label"],
                               results_stream=stream, dry_run=args.dry_run, tier_time_budget=args.tier_time_budget)
    finally:
        if stream is not None:
            stream.close()
    for cfg, stats in ranked[:10]:
        print(f"  {stats.p50_tf:8.1f} TF  {cfg.label}")
    return 0


if __name__ == "__main__":
    import sys

    sys.exit(main())
