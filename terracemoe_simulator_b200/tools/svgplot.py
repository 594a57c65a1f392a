"""A small dependency-free SVG chart writer (lines, markers, bars, heat maps, reference lines).

Figures are plain text and byte-for-byte reproducible: no timestamps, no random ids, fixed number
formatting.  Only what the figure generator of this package needs is implemented.
"""
from __future__ import annotations

import math

PALETTE = ["#1f77b4", "#d62728", "#2ca02c", "#ff7f0e", "#9467bd", "#8c564b", "#7f7f7f", "#17becf"]


def _fmt(v: float) -> str:
    return ("%.2f" % v).rstrip("0").rstrip(".")


def _esc(s: str) -> str:
    return str(s).replace("&", "&amp;").replace("<", "&lt;").replace(">", "&gt;")


def nice_ticks(lo: float, hi: float, n: int = 5):
    if hi <= lo:
        hi = lo + 1.0
    raw = (hi - lo) / max(n, 1)
    mag = 10 ** math.floor(math.log10(raw))
    step = min((m for m in (1, 2, 2.5, 5, 10) if m * mag >= raw), default=10) * mag
    first = math.ceil(lo / step - 1e-9) * step
    out, v = [], first
    while v <= hi + 1e-9 * step:
        out.append(round(v, 10))
        v += step
    return out


class Chart:
    """One set of axes.  ``xlog`` / ``ylog`` switch an axis to log10; ``xcats`` makes x categorical."""

    def __init__(self, title="", xlabel="", ylabel="", width=640, height=400, xlog=False,
                 ylog=False, xcats=None):
        self.title, self.xlabel, self.ylabel = title, xlabel, ylabel
        self.w, self.h, self.xlog, self.ylog = width, height, xlog, ylog
        self.xcats = list(xcats) if xcats is not None else None
        self.items, self.hlines, self.vlines, self.notes = [], [], [], []
        self.xlim = self.ylim = None

    # ---- content -----------------------------------------------------------------------------
    def line(self, xs, ys, label=None, color=None, marker=True, dash=None):
        self.items.append(("line", list(xs), list(ys), label, color, marker, dash))
        return self

    def bars(self, ys, label=None, color=None, group=0, n_groups=1):
        self.items.append(("bars", list(range(len(ys))), list(ys), label, color, group, n_groups))
        return self

    def band(self, xs, lo, hi, color=None, label=None):
        self.items.append(("band", list(xs), (list(lo), list(hi)), label, color, None, None))
        return self

    def hline(self, y, label=None, color="#555555"):
        self.hlines.append((y, label, color))
        return self

    def vline(self, x, label=None, color="#555555"):
        self.vlines.append((x, label, color))
        return self

    def note(self, text):
        self.notes.append(text)
        return self

    # ---- geometry ----------------------------------------------------------------------------
    def _tx(self, v):
        return math.log10(max(v, 1e-300)) if self.xlog else v

    def _ty(self, v):
        return math.log10(max(v, 1e-300)) if self.ylog else v

    def _ranges(self):
        xs, ys = [], []
        for kind, x, y, *_ in self.items:
            xs += x
            ys += (y[0] + y[1]) if kind == "band" else y
            if kind == "bars":
                ys.append(0.0 if not self.ylog else min(y))
        ys += [h[0] for h in self.hlines]
        xs += [v[0] for v in self.vlines]
        if self.xcats is not None:
            xr = (-0.5, len(self.xcats) - 0.5)
        else:
            xr = self.xlim or (min(xs), max(xs))
            xr = (self._tx(xr[0]), self._tx(xr[1]))
        yr = self.ylim or (min(ys), max(ys))
        yr = (self._ty(yr[0]), self._ty(yr[1]))
        pad = 0.06 * ((yr[1] - yr[0]) or 1.0)
        if self.ylim is None:
            yr = (yr[0] - (0 if any(i[0] == "bars" for i in self.items) and not self.ylog else pad),
                  yr[1] + pad)
        if xr[1] == xr[0]:
            xr = (xr[0] - 0.5, xr[1] + 0.5)
        return xr, yr

    def render(self) -> str:
        left, right, top, bottom = 64, 150, 34, 52
        pw, ph = self.w - left - right, self.h - top - bottom
        xr, yr = self._ranges()
        px = lambda v: left + (self._tx(v) - xr[0]) / (xr[1] - xr[0]) * pw        # noqa: E731
        pxc = lambda v: left + (v - xr[0]) / (xr[1] - xr[0]) * pw                 # noqa: E731
        py = lambda v: top + ph - (self._ty(v) - yr[0]) / (yr[1] - yr[0]) * ph    # noqa: E731
        o = ['<svg xmlns="http://www.w3.org/2000/svg" width="%d" height="%d" viewBox="0 0 %d %d" '
             'font-family="Helvetica,Arial,sans-serif" font-size="11">' % (self.w, self.h, self.w, self.h),
             '<rect width="100%" height="100%" fill="white"/>',
             '<text x="%d" y="18" font-size="13" font-weight="bold">%s</text>' % (left, _esc(self.title)),
             '<rect x="%d" y="%d" width="%d" height="%d" fill="none" stroke="#333"/>' % (left, top, pw, ph)]
        # ticks
        if self.ylog:
            yt = [10 ** e for e in range(math.floor(yr[0]), math.ceil(yr[1]) + 1)
                  if yr[0] - 1e-9 <= e <= yr[1] + 1e-9]
        else:
            yt = [t for t in nice_ticks(yr[0], yr[1]) if yr[0] <= t <= yr[1]]
        for t in yt:
            y = py(t)
            o.append('<line x1="%d" x2="%d" y1="%s" y2="%s" stroke="#ddd"/>' % (left, left + pw, _fmt(y), _fmt(y)))
            o.append('<text x="%d" y="%s" text-anchor="end">%s</text>' % (left - 5, _fmt(y + 4), _esc("%g" % t)))
        if self.xcats is not None:
            for i, c in enumerate(self.xcats):
                o.append('<text x="%s" y="%d" text-anchor="middle">%s</text>' % (_fmt(pxc(i)), top + ph + 15, _esc(c)))
        else:
            if self.xlog:
                xt = [10 ** e for e in range(math.floor(xr[0]), math.ceil(xr[1]) + 1)
                      if xr[0] - 1e-9 <= e <= xr[1] + 1e-9]
            else:
                xt = [t for t in nice_ticks(xr[0], xr[1]) if xr[0] <= t <= xr[1]]
            for t in xt:
                o.append('<text x="%s" y="%d" text-anchor="middle">%s</text>' % (_fmt(px(t)), top + ph + 15, _esc("%g" % t)))
        o.append('<text x="%s" y="%d" text-anchor="middle">%s</text>' % (_fmt(left + pw / 2), self.h - 12, _esc(self.xlabel)))
        o.append('<text transform="translate(14,%s) rotate(-90)" text-anchor="middle">%s</text>'
                 % (_fmt(top + ph / 2), _esc(self.ylabel)))
        legend = []
        for n, (kind, xs, ys, label, color, a, b) in enumerate(self.items):
            color = color or PALETTE[n % len(PALETTE)]
            if kind == "line":
                pos = pxc if self.xcats is not None else px
                pts = " ".join("%s,%s" % (_fmt(pos(x)), _fmt(py(y))) for x, y in zip(xs, ys))
                o.append('<polyline points="%s" fill="none" stroke="%s" stroke-width="1.6"%s/>'
                         % (pts, color, ' stroke-dasharray="%s"' % b if b else ""))
                if a:
                    for x, y in zip(xs, ys):
                        o.append('<circle cx="%s" cy="%s" r="2.6" fill="%s"/>' % (_fmt(pos(x)), _fmt(py(y)), color))
            elif kind == "bars":
                group, n_groups = a, b
                bw = 0.8 / n_groups * pw / (xr[1] - xr[0])
                base = py(10 ** yr[0]) if self.ylog else py(max(0.0, yr[0]))
                for x, y in zip(xs, ys):
                    x0 = pxc(x - 0.4 + 0.8 * group / n_groups)
                    y1 = py(y)
                    o.append('<rect x="%s" y="%s" width="%s" height="%s" fill="%s"/>'
                             % (_fmt(x0), _fmt(min(y1, base)), _fmt(bw), _fmt(abs(base - y1)), color))
            elif kind == "band":
                lo, hi = ys
                pts = [(px(x), py(v)) for x, v in zip(xs, hi)] + [(px(x), py(v)) for x, v in zip(xs[::-1], lo[::-1])]
                o.append('<polygon points="%s" fill="%s" fill-opacity="0.18" stroke="none"/>'
                         % (" ".join("%s,%s" % (_fmt(x), _fmt(y)) for x, y in pts), color))
            if label:
                legend.append((label, color))
        for y, label, color in self.hlines:
            o.append('<line x1="%d" x2="%d" y1="%s" y2="%s" stroke="%s" stroke-dasharray="5,3"/>'
                     % (left, left + pw, _fmt(py(y)), _fmt(py(y)), color))
            if label:
                legend.append((label, color))
        for x, label, color in self.vlines:
            o.append('<line x1="%s" x2="%s" y1="%d" y2="%d" stroke="%s" stroke-dasharray="5,3"/>'
                     % (_fmt(px(x)), _fmt(px(x)), top, top + ph, color))
            if label:
                legend.append((label, color))
        for i, (label, color) in enumerate(legend):
            y = top + 10 + 15 * i
            o.append('<rect x="%d" y="%d" width="10" height="10" fill="%s"/>' % (left + pw + 10, y - 9, color))
            o.append('<text x="%d" y="%d">%s</text>' % (left + pw + 24, y, _esc(label)))
        for i, text in enumerate(self.notes):
            o.append('<text x="%d" y="%d" fill="#444">%s</text>' % (left + 6, top + 14 + 13 * i, _esc(text)))
        o.append("</svg>")
        return "\n".join(o) + "\n"


def heatmap(grid, xlabels, ylabels, title="", xlabel="", ylabel="", center=1.0, width=640,
            height=400) -> str:
    """Diverging heat map around ``center`` (blue below, red above) with the values printed."""
    left, top, right, bottom = 80, 34, 20, 52
    n_r, n_c = len(grid), len(grid[0])
    cw, ch = (width - left - right) / n_c, (height - top - bottom) / n_r
    span = max(max(abs(v - center) for v in row) for row in grid) or 1.0
    o = ['<svg xmlns="http://www.w3.org/2000/svg" width="%d" height="%d" viewBox="0 0 %d %d" '
         'font-family="Helvetica,Arial,sans-serif" font-size="11">' % (width, height, width, height),
         '<rect width="100%" height="100%" fill="white"/>',
         '<text x="%d" y="18" font-size="13" font-weight="bold">%s</text>' % (left, _esc(title))]
    for r, row in enumerate(grid):
        for c, v in enumerate(row):
            f = max(-1.0, min(1.0, (v - center) / span))
            if f >= 0:
                rgb = (255, int(255 - 150 * f), int(255 - 170 * f))
            else:
                rgb = (int(255 + 170 * f), int(255 + 120 * f), 255)
            o.append('<rect x="%s" y="%s" width="%s" height="%s" fill="rgb(%d,%d,%d)" stroke="white"/>'
                     % (_fmt(left + c * cw), _fmt(top + r * ch), _fmt(cw), _fmt(ch), *rgb))
            o.append('<text x="%s" y="%s" text-anchor="middle">%s</text>'
                     % (_fmt(left + (c + 0.5) * cw), _fmt(top + (r + 0.5) * ch + 4), "%.2f" % v))
    for c, lab in enumerate(xlabels):
        o.append('<text x="%s" y="%s" text-anchor="middle">%s</text>'
                 % (_fmt(left + (c + 0.5) * cw), _fmt(height - bottom + 15), _esc(lab)))
    for r, lab in enumerate(ylabels):
        o.append('<text x="%d" y="%s" text-anchor="end">%s</text>' % (left - 6, _fmt(top + (r + 0.5) * ch + 4), _esc(lab)))
    o.append('<text x="%s" y="%d" text-anchor="middle">%s</text>' % (_fmt(left + (width - left - right) / 2), height - 12, _esc(xlabel)))
    o.append('<text transform="translate(14,%s) rotate(-90)" text-anchor="middle">%s</text>'
             % (_fmt(top + (height - top - bottom) / 2), _esc(ylabel)))
    o.append("</svg>")
    return "\n".join(o) + "\n"
