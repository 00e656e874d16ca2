"""Visualization without external plotting libraries: SVG line charts of training histories, tensor heat-maps,
histograms, computation-graph drawings (DOT and SVG), HTML dashboards
(src/visualization/plotting.rs:13-240, tensor_viz.rs, graph_viz.rs, utils.rs:11-420).

Everything returns a string (SVG / HTML / DOT) and ``save_plot`` writes it, as in the reference, so plots work
headless.  Tensors are reduced on their device; only the few hundred numbers that are drawn reach the host.
"""
from __future__ import annotations

import html
import os
import time
from dataclasses import dataclass, field
from enum import Enum
from typing import Dict, List, Optional, Sequence, Tuple

import torch


class PlotFormat(Enum):
    SVG = "svg"
    HTML = "html"
    DOT = "dot"

    def extension(self) -> str:
        return self.value

    def mime_type(self) -> str:
        return {"svg": "image/svg+xml", "html": "text/html", "dot": "text/vnd.graphviz"}[self.value]


class PlotStyle(Enum):
    """Line, scatter or bar rendering of a series."""

    LINE = "line"
    SCATTER = "scatter"
    BAR = "bar"


class ChartType(Enum):
    """Chart kinds the plotters draw (src/visualization/plotting.rs)."""

    LOSS = "loss"
    ACCURACY = "accuracy"
    LEARNING_RATE = "learning_rate"
    CUSTOM = "custom"


@dataclass
class PlotConfig:
    width: int = 800
    height: int = 480
    title: str = ""
    xlabel: str = "epoch"
    ylabel: str = ""
    style: PlotStyle = PlotStyle.LINE
    grid: bool = True
    legend: bool = True
    log_y: bool = False


@dataclass
class PlotMetadata:
    title: str = ""
    author: str = ""
    created: float = field(default_factory=time.time)
    tags: List[str] = field(default_factory=list)


@dataclass
class PlotData:
    x: List[float]
    y: List[float]
    label: str = ""
    color: Optional[str] = None


class ColorPalette:
    @staticmethod
    def categorical() -> List[str]:
        return ["#1f77b4", "#ff7f0e", "#2ca02c", "#d62728", "#9467bd", "#8c564b", "#e377c2", "#7f7f7f", "#bcbd22", "#17becf"]

    @staticmethod
    def sequential_blues() -> List[str]:
        return ["#f7fbff", "#deebf7", "#c6dbef", "#9ecae1", "#6baed6", "#4292c6", "#2171b5", "#08519c", "#08306b"]

    @staticmethod
    def diverging_red_blue() -> List[str]:
        return ["#b2182b", "#d6604d", "#f4a582", "#fddbc7", "#f7f7f7", "#d1e5f0", "#92c5de", "#4393c3", "#2166ac"]

    @staticmethod
    def get_categorical_color(index: int) -> str:
        p = ColorPalette.categorical()
        return p[index % len(p)]

    @staticmethod
    def get_sequential_color(value: float) -> str:
        p = ColorPalette.sequential_blues()
        return p[min(len(p) - 1, max(0, int(value * (len(p) - 1) + 0.5)))]

    @staticmethod
    def diverging(value: float) -> str:
        """``value`` in [-1, 1] -> interpolated red-white-blue."""
        v = max(-1.0, min(1.0, value))
        if v < 0:
            r, g, b = 255, int(255 * (1 + v)), int(255 * (1 + v))
        else:
            r, g, b = int(255 * (1 - v)), int(255 * (1 - v)), 255
        return f"#{r:02x}{g:02x}{b:02x}"


def _axes(cfg: PlotConfig, xmin, xmax, ymin, ymax) -> Tuple[List[str], callable, callable]:
    ml, mr, mt, mb = 60, 20, 40, 50
    pw, ph = cfg.width - ml - mr, cfg.height - mt - mb
    if xmax == xmin:
        xmax = xmin + 1
    if ymax == ymin:
        ymax = ymin + 1
    sx = lambda x: ml + (x - xmin) / (xmax - xmin) * pw
    sy = lambda y: mt + ph - (y - ymin) / (ymax - ymin) * ph
    out = [f'<svg xmlns="http://www.w3.org/2000/svg" width="{cfg.width}" height="{cfg.height}" viewBox="0 0 {cfg.width} {cfg.height}">',
           f'<rect width="{cfg.width}" height="{cfg.height}" fill="white"/>',
           f'<text x="{cfg.width / 2}" y="24" text-anchor="middle" font-size="16" font-family="sans-serif">{html.escape(cfg.title)}</text>']
    for i in range(6):
        fx, fy = xmin + (xmax - xmin) * i / 5, ymin + (ymax - ymin) * i / 5
        if cfg.grid:
            out.append(f'<line x1="{sx(fx):.1f}" y1="{mt}" x2="{sx(fx):.1f}" y2="{mt + ph}" stroke="#e0e0e0"/>')
            out.append(f'<line x1="{ml}" y1="{sy(fy):.1f}" x2="{ml + pw}" y2="{sy(fy):.1f}" stroke="#e0e0e0"/>')
        out.append(f'<text x="{sx(fx):.1f}" y="{mt + ph + 18}" text-anchor="middle" font-size="11" font-family="sans-serif">{fx:.3g}</text>')
        out.append(f'<text x="{ml - 6}" y="{sy(fy) + 4:.1f}" text-anchor="end" font-size="11" font-family="sans-serif">{fy:.3g}</text>')
    out.append(f'<rect x="{ml}" y="{mt}" width="{pw}" height="{ph}" fill="none" stroke="black"/>')
    out.append(f'<text x="{ml + pw / 2}" y="{cfg.height - 10}" text-anchor="middle" font-size="12" font-family="sans-serif">{html.escape(cfg.xlabel)}</text>')
    out.append(f'<text x="16" y="{mt + ph / 2}" text-anchor="middle" font-size="12" font-family="sans-serif" transform="rotate(-90 16 {mt + ph / 2})">{html.escape(cfg.ylabel)}</text>')
    return out, sx, sy


def line_chart(series: Sequence[PlotData], cfg: Optional[PlotConfig] = None) -> str:
    import math
    cfg = cfg or PlotConfig()
    tr = (lambda v: math.log10(max(v, 1e-12))) if cfg.log_y else (lambda v: v)
    xs = [x for s in series for x in s.x] or [0, 1]
    ys = [tr(y) for s in series for y in s.y] or [0, 1]
    out, sx, sy = _axes(cfg, min(xs), max(xs), min(ys), max(ys))
    for i, s in enumerate(series):
        col = s.color or ColorPalette.get_categorical_color(i)
        pts = [(sx(x), sy(tr(y))) for x, y in zip(s.x, s.y)]
        if cfg.style is PlotStyle.LINE and len(pts) > 1:
            out.append(f'<polyline fill="none" stroke="{col}" stroke-width="2" points="' + " ".join(f"{a:.1f},{b:.1f}" for a, b in pts) + '"/>')
        elif cfg.style is PlotStyle.BAR:
            w = max(2.0, (cfg.width - 80) / max(1, len(pts)) * 0.8)
            base = sy(min(ys))
            out += [f'<rect x="{a - w / 2:.1f}" y="{b:.1f}" width="{w:.1f}" height="{max(0.0, base - b):.1f}" fill="{col}"/>' for a, b in pts]
        else:
            out += [f'<circle cx="{a:.1f}" cy="{b:.1f}" r="3" fill="{col}"/>' for a, b in pts]
        if cfg.legend and s.label:
            out.append(f'<rect x="{cfg.width - 150}" y="{48 + 18 * i}" width="12" height="12" fill="{col}"/>')
            out.append(f'<text x="{cfg.width - 132}" y="{59 + 18 * i}" font-size="12" font-family="sans-serif">{html.escape(s.label)}</text>')
    return "\n".join(out + ["</svg>"])


class TrainingPlotter:
    def __init__(self, config: Optional[PlotConfig] = None, metadata: Optional[PlotMetadata] = None):
        self.config, self.metadata = config or PlotConfig(), metadata or PlotMetadata()

    def with_config(self, config: PlotConfig) -> "TrainingPlotter":
        self.config = config
        return self

    def with_metadata(self, metadata: PlotMetadata) -> "TrainingPlotter":
        self.metadata = metadata
        return self

    @staticmethod
    def _hist(history, key: str) -> List[float]:
        v = history[key] if isinstance(history, dict) else getattr(history, key, None)
        return [float(x) for x in (v or [])]

    def plot_training_curves(self, history) -> str:
        """``history``: a mapping / object with ``train_loss`` and optionally ``val_loss`` lists."""
        series = []
        for key, label in (("train_loss", "train"), ("val_loss", "validation")):
            y = self._hist(history, key)
            if y:
                series.append(PlotData(list(range(1, len(y) + 1)), y, label))
        cfg = PlotConfig(**{**self.config.__dict__, "title": self.config.title or "Training curves", "ylabel": "loss"})
        return line_chart(series, cfg)

    def plot_loss_comparison(self, runs: Dict[str, Sequence[float]]) -> str:
        series = [PlotData(list(range(1, len(v) + 1)), [float(x) for x in v], k) for k, v in runs.items()]
        cfg = PlotConfig(**{**self.config.__dict__, "title": self.config.title or "Loss comparison", "ylabel": "loss"})
        return line_chart(series, cfg)

    def plot_metrics_timeline(self, metrics: Dict[str, Sequence[float]]) -> str:
        series = [PlotData(list(range(1, len(v) + 1)), [float(x) for x in v], k) for k, v in metrics.items()]
        cfg = PlotConfig(**{**self.config.__dict__, "title": self.config.title or "Metrics", "ylabel": "value"})
        return line_chart(series, cfg)

    def save_plot(self, content: str, path: str) -> None:
        save_plot(content, path)


class TensorVisualizer:
    def heatmap(self, t: torch.Tensor, title: str = "", max_cells: int = 64, cell: int = 10) -> str:
        """2-D heat-map; larger matrices are average-pooled on their device down to ``max_cells`` per side."""
        m = t.detach().float()
        m = m.reshape(m.shape[0], -1) if m.dim() != 2 else m
        if max(m.shape) > max_cells:
            oh, ow = min(m.shape[0], max_cells), min(m.shape[1], max_cells)
            m = torch.nn.functional.adaptive_avg_pool2d(m[None, None], (oh, ow))[0, 0]
        scale = float(m.abs().max()) or 1.0
        vals = (m / scale).cpu().tolist()
        h, w = len(vals), len(vals[0])
        out = [f'<svg xmlns="http://www.w3.org/2000/svg" width="{w * cell}" height="{h * cell + 20}">',
               f'<text x="2" y="14" font-size="12" font-family="sans-serif">{html.escape(title)}</text>']
        for i, row in enumerate(vals):
            for j, v in enumerate(row):
                out.append(f'<rect x="{j * cell}" y="{i * cell + 20}" width="{cell}" height="{cell}" fill="{ColorPalette.diverging(v)}"/>')
        return "\n".join(out + ["</svg>"])

    def histogram(self, t: torch.Tensor, bins: int = 40, title: str = "") -> str:
        f = t.detach().float().reshape(-1)
        lo, hi = float(f.min()), float(f.max())
        counts = torch.histc(f, bins=bins, min=lo, max=hi).cpu().tolist()
        xs = [lo + (hi - lo) * (i + 0.5) / bins for i in range(bins)]
        return line_chart([PlotData(xs, counts, "count")], PlotConfig(title=title or "histogram", xlabel="value", ylabel="count", style=PlotStyle.BAR, legend=False))

    def stats(self, t: torch.Tensor) -> Dict[str, float]:
        f = t.detach().float()
        return {"mean": float(f.mean()), "std": float(f.std()) if f.numel() > 1 else 0.0, "min": float(f.min()), "max": float(f.max()),
                "sparsity": float((f == 0).float().mean()), "numel": f.numel()}


class TensorStats(TensorVisualizer):
    """``TensorStats(tensor)`` of the Python binding (src/python/visualization.rs:300-372): ``compute_stats()`` then
    ``get_stats()`` -> count / mean / std / min / max / median / q25 / q75, ``plot_stats(save_path)``.  Without a tensor
    it is the plain :class:`TensorVisualizer`."""

    def __init__(self, tensor=None):
        self.tensor = None if tensor is None else _raw_tensor(tensor)
        self._stats: Optional[Dict[str, float]] = None

    def compute_stats(self) -> None:
        if self.tensor is None or self.tensor.numel() == 0:
            raise ValueError("Cannot compute statistics for empty tensor")
        f = self.tensor.detach().double().flatten()
        srt = f.sort().values
        n = f.numel()
        self._stats = {"count": float(n), "mean": float(f.mean()), "std": float(f.var(unbiased=False).sqrt()), "min": float(srt[0]),
                       "max": float(srt[-1]), "median": float(srt[n // 2]), "q25": float(srt[n // 4]), "q75": float(srt[3 * n // 4])}

    def get_stats(self) -> Dict[str, float]:
        if self._stats is None:
            raise RuntimeError("Statistics not computed. Call compute_stats() first.")
        return dict(self._stats)

    def plot_stats(self, save_path: Optional[str] = None) -> str:
        """Histogram of the values with the computed mean / median in the title; written to ``save_path`` when given."""
        st = self.get_stats()
        svg = self.histogram(self.tensor, title=f"mean {st['mean']:.4g}  median {st['median']:.4g}  std {st['std']:.4g}")
        if save_path:
            save_plot(svg, save_path)
        return svg

    def __repr__(self) -> str:
        return f"TensorStats(computed={self._stats is not None})"


def _raw_tensor(t) -> torch.Tensor:
    if isinstance(t, torch.Tensor):
        return t
    inner = getattr(t, "tensor", None)
    if isinstance(inner, torch.Tensor):
        return inner
    inner = getattr(t, "data", None)
    return inner if isinstance(inner, torch.Tensor) else torch.as_tensor(t, dtype=torch.float32)


class GraphVisualizer:
    """Autograd-graph and module-tree drawings."""

    def autograd_dot(self, output: torch.Tensor, max_nodes: int = 500) -> str:
        lines, seen = ["digraph autograd {", "  rankdir=BT;", '  node [shape=box, fontname="sans-serif"];'], {}

        def nid(fn):
            if fn not in seen:
                seen[fn] = f"n{len(seen)}"
                lines.append(f'  {seen[fn]} [label="{type(fn).__name__}"];')
            return seen[fn]
        stack = [output.grad_fn] if output.grad_fn is not None else []
        while stack and len(seen) < max_nodes:
            fn = stack.pop()
            a = nid(fn)
            for nxt, _ in fn.next_functions:
                if nxt is not None:
                    new = nxt not in seen
                    lines.append(f"  {nid(nxt)} -> {a};")
                    if new:
                        stack.append(nxt)
        return "\n".join(lines + ["}"])

    def module_dot(self, module: torch.nn.Module) -> str:
        lines = ["digraph model {", '  node [shape=box, fontname="sans-serif"];']
        ids = {}
        for name, m in module.named_modules():
            ids[name] = f"m{len(ids)}"
            n_params = sum(p.numel() for p in m.parameters(recurse=False))
            lines.append(f'  {ids[name]} [label="{name or "model"}\\n{type(m).__name__}' + (f"\\n{n_params:,} params" if n_params else "") + '"];')
            if name:
                parent = name.rsplit(".", 1)[0] if "." in name else ""
                lines.append(f"  {ids[parent]} -> {ids[name]};")
        return "\n".join(lines + ["}"])

    def module_svg(self, module: torch.nn.Module, width: int = 420, row: int = 26) -> str:
        rows = [(name.count(".") + (1 if name else 0), name.rsplit(".", 1)[-1] or "model", type(m).__name__,
                 sum(p.numel() for p in m.parameters(recurse=False))) for name, m in module.named_modules()]
        out = [f'<svg xmlns="http://www.w3.org/2000/svg" width="{width}" height="{row * len(rows) + 10}">']
        for i, (depth, name, kind, n) in enumerate(rows):
            x = 8 + 18 * depth
            out.append(f'<rect x="{x}" y="{5 + i * row}" width="{width - x - 8}" height="{row - 4}" fill="{ColorPalette.get_sequential_color(min(1.0, depth / 6))}" stroke="#555"/>')
            out.append(f'<text x="{x + 6}" y="{5 + i * row + 15}" font-size="11" font-family="sans-serif">{html.escape(name)}: {kind}{f" ({n:,})" if n else ""}</text>')
        return "\n".join(out + ["</svg>"])


class ModelVisualizer(GraphVisualizer):
    """``ModelVisualizer(layout_engine, show_shapes, show_layer_names)`` of the Python binding
    (src/python/visualization.rs:222-298) on top of :class:`GraphVisualizer`."""

    def __init__(self, layout_engine: Optional[str] = None, show_shapes: Optional[bool] = None,
                 show_layer_names: Optional[bool] = None):
        self.layout_engine = layout_engine or "dot"
        self.show_shapes = True if show_shapes is None else bool(show_shapes)
        self.show_layer_names = True if show_layer_names is None else bool(show_layer_names)

    def visualize_model(self, model_summary, save_path: Optional[str] = None, format: Optional[str] = None) -> str:
        """``model_summary``: the text of ``model.summary()`` (one box per layer row, chained top to bottom) or a
        module (its tree).  Returns Graphviz source; ``format="svg"`` returns a drawing of the chain instead."""
        if isinstance(model_summary, torch.nn.Module):
            out = self.module_svg(model_summary) if (format or "dot").lower() == "svg" else self.module_dot(model_summary)
            if save_path:
                save_plot(out, save_path)
            return out
        if True:
            rows = [ln.strip() for ln in str(model_summary).splitlines()
                    if "(" in ln and not ln.startswith(("Model:", "Layer (type)", "Total", "Compiled"))]
            lines = [f"digraph model {{", f"  layout={self.layout_engine};", "  rankdir=TB;", '  node [shape=box, fontname="sans-serif"];']
            for i, r in enumerate(rows):
                parts = r.split()
                label = (parts[0] + " " + parts[1] if self.show_layer_names and len(parts) > 1 else parts[1] if len(parts) > 1 else parts[0])
                if self.show_shapes and "(None" in r:
                    label += "\\n" + r[r.index("(None"):r.index(")", r.index("(None")) + 1]
                lines.append(f'  l{i} [label="{label}"];')
            lines += [f"  l{i} -> l{i + 1};" for i in range(len(rows) - 1)] + ["}"]
            dot = "\n".join(lines)
        out = dot
        if (format or "dot").lower() == "svg":
            h = 40 * max(1, len(rows)) + 20
            body = [f'<svg xmlns="http://www.w3.org/2000/svg" width="420" height="{h}">', f'<rect width="420" height="{h}" fill="white"/>']
            for i, r in enumerate(rows):
                body.append(f'<rect x="10" y="{10 + 40 * i}" width="400" height="28" fill="#deebf7" stroke="#2171b5"/>')
                body.append(f'<text x="18" y="{29 + 40 * i}" font-size="12" font-family="monospace">{html.escape(r[:56])}</text>')
                if i:
                    body.append(f'<line x1="210" y1="{40 * i - 2}" x2="210" y2="{10 + 40 * i}" stroke="black"/>')
            out = "\n".join(body + ["</svg>"])
        if save_path:
            save_plot(out, save_path)
        return out

    def plot_attention_heatmap(self, attention_weights, tokens: Optional[Sequence[str]] = None, title: Optional[str] = None,
                               save_path: Optional[str] = None) -> str:
        """``[T, S]`` attention weights (or ``[..., T, S]``: leading dimensions averaged) as a heat-map with token labels."""
        w = _raw_tensor(attention_weights).detach().float()
        while w.dim() > 2:
            w = w.mean(0)
        if w.dim() != 2:
            raise ValueError("attention weights must have at least two dimensions")
        T, S = w.shape
        if tokens is not None and len(tokens) not in (T, S):
            raise ValueError(f"{len(tokens)} tokens for a {T} x {S} attention map")
        cell, left, top = 22, 90, 60
        scale = float(w.max()) or 1.0
        vals = (w / scale).cpu().tolist()
        out = [f'<svg xmlns="http://www.w3.org/2000/svg" width="{left + S * cell + 10}" height="{top + T * cell + 10}">',
               f'<rect width="100%" height="100%" fill="white"/>',
               f'<text x="{left}" y="18" font-size="14" font-family="sans-serif">{html.escape(title or "Attention")}</text>']
        for i in range(T):
            for j in range(S):
                out.append(f'<rect x="{left + j * cell}" y="{top + i * cell}" width="{cell}" height="{cell}" fill="{ColorPalette.get_sequential_color(vals[i][j])}"/>')
        if tokens is not None:
            for i in range(T):
                out.append(f'<text x="{left - 4}" y="{top + i * cell + 15}" text-anchor="end" font-size="11" font-family="sans-serif">{html.escape(str(tokens[i % len(tokens)]))}</text>')
            for j in range(S):
                x = left + j * cell + 14
                out.append(f'<text x="{x}" y="{top - 4}" font-size="11" font-family="sans-serif" transform="rotate(-60 {x} {top - 4})">{html.escape(str(tokens[j % len(tokens)]))}</text>')
        svg = "\n".join(out + ["</svg>"])
        if save_path:
            save_plot(svg, save_path)
        return svg

    def __repr__(self) -> str:
        return f"ModelVisualizer(layout_engine='{self.layout_engine}', show_shapes={self.show_shapes})"


class Plotter(TrainingPlotter):
    """``Plotter(backend, style, figure_size, dpi)`` of the Python binding (src/python/visualization.rs:11-220).  Every
    method returns the SVG text and writes it to ``save_path`` when one is given (the reference prints a description of
    the plot instead of drawing it)."""

    def __init__(self, backend=None, style: Optional[str] = None, figure_size: Optional[Tuple[int, int]] = None,
                 dpi: Optional[int] = None, config: Optional[PlotConfig] = None, metadata: Optional[PlotMetadata] = None):
        if isinstance(backend, PlotConfig):                           # TrainingPlotter(config, metadata) order
            config, backend = backend, None
        if isinstance(style, PlotMetadata):
            metadata, style = style, None
        self.backend, self.style_name, self.dpi = backend or "svg", style or "default", int(dpi or 100)
        self.figure_size = tuple(figure_size or (10, 6))
        cfg = config or PlotConfig(width=int(self.figure_size[0] * 80), height=int(self.figure_size[1] * 80))
        super().__init__(cfg, metadata)

    def _cfg(self, **kw) -> PlotConfig:
        return PlotConfig(**{**self.config.__dict__, **{k: v for k, v in kw.items() if v is not None}})

    def _done(self, svg: str, save_path: Optional[str]) -> str:
        if save_path:
            save_plot(svg, save_path)
        return svg

    def plot_training_history(self, history, save_path: Optional[str] = None, show_validation: Optional[bool] = None) -> str:
        show_val = True if show_validation is None else bool(show_validation)
        tr = [float(v) for v in (history.train_loss() if callable(getattr(history, "train_loss", None)) else history["train_loss"])]
        va = [float(v) for v in (history.val_loss() if callable(getattr(history, "val_loss", None)) else history.get("val_loss", []))]
        series = [PlotData(list(range(1, len(tr) + 1)), tr, "train")]
        if show_val and va:
            series.append(PlotData(list(range(1, len(va) + 1)), va, "validation"))
        return self._done(line_chart(series, self._cfg(title=self.config.title or "Training history", ylabel="loss")), save_path)

    def plot_tensor_as_image(self, tensor, title: Optional[str] = None, colormap: Optional[str] = None,
                             save_path: Optional[str] = None) -> str:
        return self._done(TensorVisualizer().heatmap(_raw_tensor(tensor), title or "Tensor"), save_path)

    def plot_multiple_tensors(self, tensors, titles: Optional[Sequence[str]] = None, layout: Optional[Tuple[int, int]] = None,
                              save_path: Optional[str] = None) -> str:
        n = len(tensors)
        if titles is not None and len(titles) != n:
            raise ValueError(f"{len(titles)} titles for {n} tensors")
        rows, cols = layout or (1, n)
        if rows * cols < n:
            raise ValueError(f"layout {rows} x {cols} holds fewer than {n} tensors")
        plots = [((titles[i] if titles else f"tensor {i}"), TensorVisualizer().heatmap(_raw_tensor(t))) for i, t in enumerate(tensors)]
        cells = []
        for r in range(rows):
            row = "".join(f"<td style='padding:6px;vertical-align:top'><div style='font-family:sans-serif'>{html.escape(t)}</div>{s}</td>"
                          for t, s in plots[r * cols:(r + 1) * cols])
            cells.append(f"<tr>{row}</tr>")
        return self._done(wrap_in_html("<table>" + "".join(cells) + "</table>", "tensors"), save_path)

    def line_plot(self, x_data, y_data, title: Optional[str] = None, xlabel: Optional[str] = None, ylabel: Optional[str] = None,
                  save_path: Optional[str] = None) -> str:
        if len(x_data) != len(y_data):
            raise ValueError("x_data and y_data must have the same length")
        cfg = self._cfg(title=title or "Line Plot", xlabel=xlabel or "x", ylabel=ylabel or "y", style=PlotStyle.LINE, legend=False)
        return self._done(line_chart([PlotData([float(v) for v in x_data], [float(v) for v in y_data])], cfg), save_path)

    def scatter_plot(self, x_data, y_data, colors=None, sizes=None, title: Optional[str] = None, save_path: Optional[str] = None) -> str:
        if len(x_data) != len(y_data):
            raise ValueError("x_data and y_data must have the same length")
        for name, extra in (("colors", colors), ("sizes", sizes)):
            if extra is not None and len(extra) != len(x_data):
                raise ValueError(f"{name} must have one entry per point")
        cfg = self._cfg(title=title or "Scatter Plot", xlabel="x", ylabel="y", legend=False)
        xs, ys = [float(v) for v in x_data], [float(v) for v in y_data]
        out, sx, sy = _axes(cfg, min(xs, default=0.0), max(xs, default=1.0), min(ys, default=0.0), max(ys, default=1.0))
        lo, hi = (min(colors), max(colors)) if colors else (0.0, 1.0)
        for i, (a, b) in enumerate(zip(xs, ys)):
            col = ColorPalette.get_sequential_color(0.3 + 0.7 * ((colors[i] - lo) / (hi - lo) if hi > lo else 1.0)) if colors else ColorPalette.get_categorical_color(0)
            out.append(f'<circle cx="{sx(a):.1f}" cy="{sy(b):.1f}" r="{float(sizes[i]) if sizes else 3.0:.1f}" fill="{col}"/>')
        return self._done("\n".join(out + ["</svg>"]), save_path)

    def histogram(self, data, bins: Optional[int] = None, title: Optional[str] = None, xlabel: Optional[str] = None,
                  ylabel: Optional[str] = None, save_path: Optional[str] = None) -> str:
        t = _raw_tensor(data).float().flatten()
        if t.numel() == 0:
            raise ValueError("histogram of no data")
        nb = int(bins or 30)
        lo, hi = float(t.min()), float(t.max())
        counts = torch.histc(t, bins=nb, min=lo, max=hi if hi > lo else lo + 1).tolist()
        xs = [lo + (max(hi - lo, 1.0 if hi == lo else hi - lo)) * (i + 0.5) / nb for i in range(nb)]
        cfg = self._cfg(title=title or "Histogram", xlabel=xlabel or "Value", ylabel=ylabel or "Frequency", style=PlotStyle.BAR, legend=False)
        return self._done(line_chart([PlotData(xs, counts, "count")], cfg), save_path)

    def __repr__(self) -> str:
        return f"Plotter(backend='{self.backend}', style='{self.style_name}', figure_size={self.figure_size}, dpi={self.dpi})"


def wrap_in_html(svg: str, title: str = "plot") -> str:
    return f"<!DOCTYPE html><html><head><meta charset='utf-8'><title>{html.escape(title)}</title></head><body>{svg}</body></html>"


def create_dashboard(plots: Sequence[Tuple[str, str]]) -> str:
    cells = "".join(f"<div style='display:inline-block;margin:8px;vertical-align:top'><h3 style='font-family:sans-serif'>{html.escape(t)}</h3>{s}</div>" for t, s in plots)
    return f"<!DOCTYPE html><html><head><meta charset='utf-8'><title>dashboard</title></head><body>{cells}</body></html>"


def save_plot(content: str, path: str, fmt: Optional[PlotFormat] = None) -> None:
    if fmt is PlotFormat.HTML and not content.lstrip().lower().startswith("<!doctype"):
        content = wrap_in_html(content)
    os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
    with open(path, "w") as f:
        f.write(content)


def resize_svg(svg: str, width: int, height: int) -> str:
    import re
    svg = re.sub(r'width="\d+(\.\d+)?"', f'width="{width}"', svg, count=1)
    return re.sub(r'height="\d+(\.\d+)?"', f'height="{height}"', svg, count=1)


def generate_filename(base: str, fmt: PlotFormat, timestamp: bool = False) -> str:
    return f"{base}_{time.strftime('%Y%m%d_%H%M%S')}.{fmt.extension()}" if timestamp else f"{base}.{fmt.extension()}"
