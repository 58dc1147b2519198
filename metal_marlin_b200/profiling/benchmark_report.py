"""Aggregate benchmark JSON lines / files into one table and a Markdown report.

Inputs are what ``bench.py``, ``bench/serving_load.py``, ``profiling.kernel_bench`` and the quality tools print: one JSON
object per line or per file.  ``aggregate_results`` flattens them into a :class:`pandas.DataFrame` (one row per
measurement), ``generate_markdown_report`` renders the summary, per-model breakdown and a baseline comparison.

Parity: reference ``metal_marlin/benchmark_report.py:56-847`` (``BenchmarkEntry``, ``aggregate_results``,
``generate_markdown_report``, ``generate_results_file``, ``main``); plots are left to the caller (no display stack here).
"""
from __future__ import annotations

import argparse
import json
from dataclasses import asdict, dataclass
from pathlib import Path
from typing import Any, Dict, Iterable, List, Optional, Union

import pandas as pd


@dataclass
class BenchmarkEntry:
    source: str
    model: str
    metric: str
    value: float
    unit: str = ""
    n_gpus: int = 1
    batch: Optional[int] = None
    seq_len: Optional[int] = None
    ms_per_step: Optional[float] = None
    impl: str = "ours"
    vs_baseline: Optional[float] = None
    extra: str = ""


def _entries_of(obj: Dict[str, Any], source: str) -> List[BenchmarkEntry]:
    out: List[BenchmarkEntry] = []
    if "metric" in obj and "value" in obj:          # bench.py line
        cfg = obj.get("config", {}) or {}
        model = str(cfg.get("model", obj.get("metric", ""))).split(" ")[0]
        base = dict(source=source, model=model, n_gpus=int(obj.get("n_gpus", 1)), seq_len=cfg.get("seq_len"), impl=obj.get("impl", "ours"))
        out.append(BenchmarkEntry(metric=obj["metric"], value=float(obj["value"]), unit=obj.get("unit", ""), batch=cfg.get("global_batch"),
                                  ms_per_step=obj.get("ms_per_step"), vs_baseline=obj.get("vs_baseline"), **base))
        if isinstance(obj.get("e2e"), dict) and "value" in obj["e2e"]:
            out.append(BenchmarkEntry(metric=obj["metric"] + "_e2e", value=float(obj["e2e"]["value"]), unit=obj["e2e"].get("unit", ""),
                                      batch=cfg.get("global_batch"), ms_per_step=obj["e2e"].get("ms_per_step"), **base))
        if "ttft_ms_p50" in obj:
            out.append(BenchmarkEntry(metric="ttft_ms_p50", value=float(obj["ttft_ms_p50"]), unit="ms", batch=cfg.get("global_batch"), **base))
        ex = obj.get("extra") or {}
        if "bs32_tok_s" in ex:
            out.append(BenchmarkEntry(metric="decode_tok_s_bs32", value=float(ex["bs32_tok_s"]), unit="tok/s", batch=32,
                                      ms_per_step=ex.get("bs32_ms_per_step"), **base))
        tp = obj.get("tp") or {}
        if "tok_s" in tp:
            out.append(BenchmarkEntry(metric="decode_tok_s_tp", value=float(tp["tok_s"]), unit="tok/s", batch=tp.get("global_batch"),
                                      ms_per_step=tp.get("ms_per_step"), extra=str(tp.get("parallelism", "")), **base))
    elif "results" in obj and isinstance(obj["results"], dict):     # kernel_bench summary
        for k, r in obj["results"].items():
            val = r.get("us", r.get("us_per_launch_in_graph"))
            if val is not None:
                out.append(BenchmarkEntry(source=source, model="kernel", metric=k, value=float(val), unit="us", batch=obj.get("batch"),
                                          seq_len=obj.get("ctx"), extra=json.dumps({x: r[x] for x in r if x not in ("us",)})))
    elif "output_tok_s" in obj:                                     # serving load
        for k in ("ttft_ms_p50", "ttft_ms_p99", "latency_ms_p50", "latency_ms_p99", "output_tok_s"):
            if k in obj:
                out.append(BenchmarkEntry(source=source, model=str(obj.get("model", "")), metric="serving_" + k, value=float(obj[k]),
                                          unit="tok/s" if k.endswith("tok_s") else "ms", extra=f"rate={obj.get('rate_req_s')}"))
    elif "perplexity" in obj or "ppl" in obj:
        out.append(BenchmarkEntry(source=source, model=str(obj.get("model", "")), metric="perplexity",
                                  value=float(obj.get("perplexity", obj.get("ppl"))), extra=str(obj.get("format", ""))))
    return out


def parse_lines(lines: Iterable[str], source: str = "") -> List[BenchmarkEntry]:
    out: List[BenchmarkEntry] = []
    for ln in lines:
        ln = ln.strip()
        if not ln.startswith("{"):
            continue
        try:
            out += _entries_of(json.loads(ln), source)
        except (ValueError, TypeError):
            continue
    return out


def aggregate_results(results_dir: Union[str, Path]) -> pd.DataFrame:
    """Every ``*.json`` / ``*.jsonl`` / ``*.log`` file under ``results_dir`` -> one row per measurement."""
    entries: List[BenchmarkEntry] = []
    for p in sorted(Path(results_dir).rglob("*")):
        if p.suffix in (".json", ".jsonl", ".log") and p.is_file():
            text = p.read_text(errors="replace")
            got = parse_lines(text.splitlines(), p.name)
            if not got and p.suffix == ".json":
                try:
                    got = _entries_of(json.loads(text), p.name)
                except (ValueError, TypeError):
                    got = []
            entries += got
    return pd.DataFrame([asdict(e) for e in entries], columns=list(BenchmarkEntry.__dataclass_fields__))


def generate_markdown_report(df: pd.DataFrame, title: str = "Benchmark report") -> str:
    lines = [f"# {title}", "", f"{len(df)} measurements from {df['source'].nunique() if len(df) else 0} files.", ""]
    if not len(df):
        return "\n".join(lines)
    lines += ["## Summary (best value per model and metric)", "", "| model | metric | impl | GPUs | batch | value | unit | ms/step | vs baseline |",
              "|---|---|---|---|---|---|---|---|---|"]
    time_like = df["unit"].isin(["ms", "us"])
    for (model, metric, impl, gpus), g in df.groupby(["model", "metric", "impl", "n_gpus"], dropna=False):
        r = g.loc[g["value"].idxmin()] if time_like[g.index].all() else g.loc[g["value"].idxmax()]
        f = lambda v, nd=2: "" if v is None or (isinstance(v, float) and v != v) else (f"{v:.{nd}f}" if isinstance(v, float) else str(v))
        lines.append(f"| {model} | {metric} | {impl} | {gpus} | {f(r['batch'])} | {f(float(r['value']))} | {r['unit']} | {f(r['ms_per_step'], 3)} | {f(r['vs_baseline'])} |")
    ours = df[(df["impl"] == "ours") & ~time_like]
    base = df[(df["impl"] != "ours") & ~time_like]
    if len(ours) and len(base):
        lines += ["", "## Against the baselines measured on the same box", "", "| model | metric | GPUs | ours | baseline (impl) | ratio |", "|---|---|---|---|---|---|"]
        for (model, metric, gpus), g in ours.groupby(["model", "metric", "n_gpus"]):
            b = base[(base["model"] == model) & (base["metric"] == metric) & (base["n_gpus"] == gpus)]
            for impl, gb in b.groupby("impl"):
                o, bb = float(g["value"].max()), float(gb["value"].max())
                lines.append(f"| {model} | {metric} | {gpus} | {o:.2f} | {bb:.2f} ({impl}) | {o / bb:.2f} x |" if bb else "")
    return "\n".join(lines) + "\n"


def generate_results_file(results_dir: Union[str, Path], output_dir: Optional[Union[str, Path]] = None) -> Path:
    df = aggregate_results(results_dir)
    out_dir = Path(output_dir or results_dir)
    out_dir.mkdir(parents=True, exist_ok=True)
    df.to_csv(out_dir / "results.csv", index=False)
    path = out_dir / "RESULTS.md"
    path.write_text(generate_markdown_report(df))
    return path


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("results_dir")
    ap.add_argument("--output-dir", default=None)
    a = ap.parse_args(argv)
    print(generate_results_file(a.results_dir, a.output_dir))


if __name__ == "__main__":
    main()
