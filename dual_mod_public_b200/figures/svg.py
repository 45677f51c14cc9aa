"""A small chart writer: line plots, heat maps and panel grids as SVG text, no plotting library needed.

The reference renders its figures with matplotlib's Agg backend (figures/render/*.py); this image has no
matplotlib, and a figure that is a handful of poly-lines or a grid of coloured cells needs none.  `Axes`
maps data to pixels with a linear or log2 scale per axis and collects SVG elements; `Figure` lays axes
out on a grid and writes the file.
"""

from __future__ import annotations

import math
from xml.sax.saxutils import escape

VIRIDIS = [(68, 1, 84), (72, 40, 120), (62, 74, 137), (49, 104, 142), (38, 130, 142), (31, 158, 137),
           (53, 183, 121), (109, 205, 89), (180, 222, 44), (253, 231, 37)]


def viridis(t):
    """Colour of t in [0, 1] on a ten-point viridis ramp, as #rrggbb."""
    t = min(1.0, max(0.0, float(t))) * (len(VIRIDIS) - 1)
    i = min(len(VIRIDIS) - 2, int(t))
    f = t - i
    c = [round(a + (b - a) * f) for a, b in zip(VIRIDIS[i], VIRIDIS[i + 1])]
    return "#%02x%02x%02x" % tuple(c)


class Axes:
    def __init__(self, x, y, w, h, xlim, ylim, xlog=False, ylog=False, title="", xlabel="", ylabel=""):
        self.x, self.y, self.w, self.h = x, y, w, h
        self.xlim, self.ylim, self.xlog, self.ylog = xlim, ylim, xlog, ylog
        self.items, self.legend = [], []
        self.title, self.xlabel, self.ylabel = title, xlabel, ylabel
        self.xticks, self.yticks = None, None

    @staticmethod
    def _t(v, lim, log):
        if log:
            v, lim = math.log2(max(v, 1e-300)), (math.log2(lim[0]), math.log2(lim[1]))
        return (v - lim[0]) / (lim[1] - lim[0])

    def px(self, v):
        return self.x + self.w * self._t(v, self.xlim, self.xlog)

    def py(self, v):
        return self.y + self.h * (1.0 - self._t(v, self.ylim, self.ylog))

    def line(self, xs, ys, color="#000", width=2.0, dash=None, marker=None, label=None, alpha=1.0):
        pts = [(self.px(a), self.py(b)) for a, b in zip(xs, ys) if b is not None and not (isinstance(b, float) and math.isnan(b))]
        if len(pts) > 1:
            d = " ".join(f"{a:.1f},{b:.1f}" for a, b in pts)
            da = f' stroke-dasharray="{dash}"' if dash else ""
            self.items.append(f'<polyline points="{d}" fill="none" stroke="{color}" stroke-width="{width}" '
                              f'stroke-opacity="{alpha}"{da} clip-path="url(#c{id(self)})"/>')
        if marker:
            for a, b in pts:
                fill = "#fff" if marker == "open" else color
                self.items.append(f'<circle cx="{a:.1f}" cy="{b:.1f}" r="3" fill="{fill}" stroke="{color}" fill-opacity="{alpha}"/>')
        if label:
            self.legend.append((label, color, dash))

    def hline(self, y, color="#999", dash="3,3", text=None):
        self.items.append(f'<line x1="{self.x}" x2="{self.x + self.w}" y1="{self.py(y):.1f}" y2="{self.py(y):.1f}" '
                          f'stroke="{color}" stroke-dasharray="{dash}"/>')
        if text:
            self.text(self.xlim[0], y, text, dy=-3, size=9, color="#666", anchor="start", dx=4)

    def span(self, x0, x1, color="#ebebeb"):
        a, b = self.px(x0), self.px(x1)
        self.items.insert(0, f'<rect x="{a:.1f}" y="{self.y}" width="{b - a:.1f}" height="{self.h}" fill="{color}"/>')

    def text(self, x, y, s, size=10, color="#000", anchor="middle", dx=0, dy=0):
        self.items.append(f'<text x="{self.px(x) + dx:.1f}" y="{self.py(y) + dy:.1f}" font-size="{size}" fill="{color}" '
                          f'text-anchor="{anchor}" font-family="sans-serif">{escape(str(s))}</text>')

    def heat(self, M, xlabels, ylabels, fmt=lambda v: f"{v:.2f}", notes=None):
        """M[i][j] in [0, 1] (None = empty) as a grid of cells, row 0 at the bottom."""
        ny, nx = len(M), len(M[0])
        cw, ch = self.w / nx, self.h / ny
        for i in range(ny):
            for j in range(nx):
                v = M[i][j]
                x0, y0 = self.x + j * cw, self.y + self.h - (i + 1) * ch
                self.items.append(f'<rect x="{x0:.1f}" y="{y0:.1f}" width="{cw:.1f}" height="{ch:.1f}" '
                                  f'fill="{viridis(v) if v is not None else "#fff"}" stroke="#fff"/>')
                if v is not None:
                    s = fmt(v) + (f" {notes[i][j]}" if notes and notes[i][j] else "")
                    self.items.append(f'<text x="{x0 + cw / 2:.1f}" y="{y0 + ch / 2 + 3:.1f}" font-size="9" text-anchor="middle" '
                                      f'font-family="sans-serif" fill="{"#000" if v > 0.6 else "#fff"}">{escape(s)}</text>')
        self.xticks = [(self.xlim[0] + (j + 0.5) * (self.xlim[1] - self.xlim[0]) / nx, str(l)) for j, l in enumerate(xlabels)]
        self.yticks = [(self.ylim[0] + (i + 0.5) * (self.ylim[1] - self.ylim[0]) / ny, str(l)) for i, l in enumerate(ylabels)]

    def _auto(self, lim, log):
        if log:
            lo, hi = math.ceil(math.log2(lim[0])), math.floor(math.log2(lim[1]))
            return [(2.0 ** e, str(int(2 ** e)) if e >= 0 else f"{2.0 ** e:g}") for e in range(lo, hi + 1)]
        step = (lim[1] - lim[0]) / 5
        mag = 10 ** math.floor(math.log10(step))
        step = min((m * mag for m in (1, 2, 5, 10) if m * mag >= step), default=step)
        v, out = math.ceil(lim[0] / step) * step, []
        while v <= lim[1] + 1e-9:
            out.append((v, f"{v:g}"))
            v += step
        return out

    def render(self):
        out = [f'<clipPath id="c{id(self)}"><rect x="{self.x}" y="{self.y}" width="{self.w}" height="{self.h}"/></clipPath>']
        out += self.items
        out.append(f'<rect x="{self.x}" y="{self.y}" width="{self.w}" height="{self.h}" fill="none" stroke="#333"/>')
        for v, l in (self.xticks if self.xticks is not None else self._auto(self.xlim, self.xlog)):
            out.append(f'<text x="{self.px(v):.1f}" y="{self.y + self.h + 13}" font-size="9" text-anchor="middle" '
                       f'font-family="sans-serif">{escape(l)}</text>')
        for v, l in (self.yticks if self.yticks is not None else self._auto(self.ylim, self.ylog)):
            out.append(f'<text x="{self.x - 5}" y="{self.py(v) + 3:.1f}" font-size="9" text-anchor="end" '
                       f'font-family="sans-serif">{escape(l)}</text>')
        cx = self.x + self.w / 2
        if self.title:
            out.append(f'<text x="{cx}" y="{self.y - 7}" font-size="11" text-anchor="middle" font-family="sans-serif">{escape(self.title)}</text>')
        if self.xlabel:
            out.append(f'<text x="{cx}" y="{self.y + self.h + 28}" font-size="10" text-anchor="middle" font-family="sans-serif">{escape(self.xlabel)}</text>')
        if self.ylabel:
            yy = self.y + self.h / 2
            out.append(f'<text x="{self.x - 34}" y="{yy}" font-size="10" text-anchor="middle" font-family="sans-serif" '
                       f'transform="rotate(-90 {self.x - 34} {yy})">{escape(self.ylabel)}</text>')
        return out


class Figure:
    def __init__(self, width, height, title=""):
        self.width, self.height, self.title, self.axes, self.extra = width, height, title, [], []

    def add(self, *a, **k):
        ax = Axes(*a, **k)
        self.axes.append(ax)
        return ax

    def legend(self, x, y, entries=None, cols=1, col_w=230):
        entries = entries if entries is not None else [e for ax in self.axes for e in ax.legend]
        seen, uniq = set(), []
        for e in entries:
            if e[0] not in seen:
                seen.add(e[0])
                uniq.append(e)
        for i, (label, color, dash) in enumerate(uniq):
            xx, yy = x + (i % cols) * col_w, y + (i // cols) * 14
            da = f' stroke-dasharray="{dash}"' if dash else ""
            self.extra.append(f'<line x1="{xx}" x2="{xx + 22}" y1="{yy}" y2="{yy}" stroke="{color}" stroke-width="2"{da}/>')
            self.extra.append(f'<text x="{xx + 27}" y="{yy + 3}" font-size="9" font-family="sans-serif">{escape(label)}</text>')

    def save(self, path):
        body = [f'<svg xmlns="http://www.w3.org/2000/svg" width="{self.width}" height="{self.height}" '
                f'viewBox="0 0 {self.width} {self.height}">', f'<rect width="{self.width}" height="{self.height}" fill="#fff"/>']
        if self.title:
            body.append(f'<text x="{self.width / 2}" y="16" font-size="12" text-anchor="middle" font-family="sans-serif">{escape(self.title)}</text>')
        for ax in self.axes:
            body += ax.render()
        body += self.extra + ["</svg>"]
        with open(path, "w") as f:
            f.write("\n".join(body))
        return path
