"""Vector PDF from the SVG subset that ``tools/svgplot.py`` emits (no plotting library needed).

Handles ``rect``, ``line``, ``polyline``, ``polygon``, ``circle`` and ``text`` (with
``text-anchor``, ``font-size``, ``font-weight``, ``fill`` and the ``translate(x,y) rotate(-90)``
transform of axis labels), colours as ``#rgb``, ``#rrggbb``, ``rgb(r,g,b)`` or ``white`` /
``none``, dash arrays and ``fill-opacity``.  Text uses the built-in Helvetica faces with their
standard advance widths, so anchors land where a browser puts them to within a pixel.  One page,
no compression, PDF 1.4.

``gen_figures`` writes a ``.pdf`` beside every ``.svg`` when ``TERRACE_FIG_PDF=1``; the
reference does the same through its plotting library (``tools/gen_figures.py:35-40``).
"""
from __future__ import annotations

import math
import re
import xml.etree.ElementTree as ET

# Helvetica advance widths (1/1000 em) for the printable ASCII range 32..126
_HELV = [278, 278, 355, 556, 556, 889, 667, 191, 333, 333, 389, 584, 278, 333, 278, 278,
         556, 556, 556, 556, 556, 556, 556, 556, 556, 556, 278, 278, 584, 584, 584, 556,
         1015, 667, 667, 722, 722, 667, 611, 778, 722, 278, 500, 667, 556, 833, 722, 778,
         667, 778, 722, 667, 611, 722, 667, 944, 667, 667, 611, 278, 278, 278, 469, 556,
         333, 556, 556, 500, 556, 556, 278, 556, 556, 222, 222, 500, 222, 833, 556, 556,
         556, 556, 333, 500, 278, 556, 500, 722, 500, 500, 500, 334, 260, 334, 584]
_NAMED = {"white": (1.0, 1.0, 1.0), "black": (0.0, 0.0, 0.0)}


def text_width(s: str, size: float, bold: bool = False) -> float:
    w = sum(_HELV[ord(c) - 32] if 32 <= ord(c) <= 126 else 556 for c in s)
    return w / 1000.0 * size * (1.06 if bold else 1.0)


def _color(v):
    """``(r, g, b)`` in 0..1, or ``None`` for ``none`` / a missing attribute."""
    if v is None:
        return None
    v = v.strip().lower()
    if v == "none":
        return None
    if v in _NAMED:
        return _NAMED[v]
    if v.startswith("#"):
        h = v[1:]
        if len(h) == 3:
            h = "".join(c * 2 for c in h)
        return tuple(int(h[i:i + 2], 16) / 255.0 for i in (0, 2, 4))
    m = re.match(r"rgb\(\s*(\d+)\s*,\s*(\d+)\s*,\s*(\d+)\s*\)", v)
    if m:
        return tuple(int(g) / 255.0 for g in m.groups())
    raise ValueError(f"unsupported colour {v!r}")


def _len(v, total: float) -> float:
    v = str(v)
    return float(v[:-1]) / 100.0 * total if v.endswith("%") else float(v)


def _n(x: float) -> str:
    s = ("%.2f" % x).rstrip("0").rstrip(".")
    return "0" if s in ("-0", "") else s


def _pdf_str(s: str) -> bytes:
    raw = s.encode("cp1252", errors="replace")
    return b"(" + raw.replace(b"\\", b"\\\\").replace(b"(", b"\\(").replace(b")", b"\\)") + b")"


class _Page:
    def __init__(self):
        self.ops = []
        self.alphas = {}           # fill opacity -> ExtGState name

    def paint(self, fill, stroke, width=1.0, dash=None, opacity=None):
        """Set the colours and return the painting operator for the current path."""
        if opacity is not None and opacity < 1.0:
            name = self.alphas.setdefault(round(opacity, 3), "GS%d" % (len(self.alphas) + 1))
            self.ops.append("/%s gs" % name)
        if fill is not None:
            self.ops.append("%s %s %s rg" % tuple(_n(c) for c in fill))
        if stroke is not None:
            self.ops.append("%s %s %s RG %s w" % (*(_n(c) for c in stroke), _n(width)))
            self.ops.append("[%s] 0 d" % " ".join(_n(float(d)) for d in re.split(r"[ ,]+", dash))
                            if dash else "[] 0 d")
        return "B" if fill is not None and stroke is not None else "f" if fill is not None \
            else "S" if stroke is not None else "n"


def convert(svg_text: str) -> bytes:
    root = ET.fromstring(svg_text)
    W, H = float(root.get("width")), float(root.get("height"))
    base_size = float(root.get("font-size", "11"))
    page = _Page()
    ops = page.ops
    ops.append("1 0 0 -1 0 %s cm" % _n(H))                # SVG coordinates: y grows downwards
    for el in root.iter():
        tag = el.tag.rsplit("}", 1)[-1]
        fill, stroke = _color(el.get("fill")), _color(el.get("stroke"))
        sw = float(el.get("stroke-width", "1"))
        dash = el.get("stroke-dasharray")
        opacity = float(el.get("fill-opacity")) if el.get("fill-opacity") else None
        if tag == "rect":
            x, y = float(el.get("x", "0")), float(el.get("y", "0"))
            w, h = _len(el.get("width"), W), _len(el.get("height"), H)
            if el.get("fill") is None:
                fill = (0.0, 0.0, 0.0)
            ops.append("q")
            op = page.paint(fill, stroke, sw, dash, opacity)
            ops.append("%s %s %s %s re %s" % (_n(x), _n(y), _n(w), _n(h), op))
            ops.append("Q")
        elif tag == "line":
            ops.append("q")
            op = page.paint(None, stroke or (0.0, 0.0, 0.0), sw, dash)
            ops.append("%s %s m %s %s l %s" % (_n(float(el.get("x1"))), _n(float(el.get("y1"))),
                                                _n(float(el.get("x2"))), _n(float(el.get("y2"))), op))
            ops.append("Q")
        elif tag in ("polyline", "polygon"):
            pts = [tuple(float(v) for v in p.split(",")) for p in el.get("points").split()]
            if len(pts) < 2:
                continue
            if tag == "polygon" and el.get("fill") is None:
                fill = (0.0, 0.0, 0.0)
            ops.append("q")
            op = page.paint(fill if tag == "polygon" else None, stroke, sw, dash, opacity)
            path = "%s %s m " % (_n(pts[0][0]), _n(pts[0][1]))
            path += " ".join("%s %s l" % (_n(x), _n(y)) for x, y in pts[1:])
            ops.append(path + (" h " if tag == "polygon" else " ") + op)
            ops.append("Q")
        elif tag == "circle":
            cx, cy, r = float(el.get("cx")), float(el.get("cy")), float(el.get("r"))
            k = 0.5523 * r
            if el.get("fill") is None:
                fill = (0.0, 0.0, 0.0)
            ops.append("q")
            op = page.paint(fill, stroke, sw, dash, opacity)
            ops.append("%s %s m %s %s %s %s %s %s c %s %s %s %s %s %s c %s %s %s %s %s %s c "
                       "%s %s %s %s %s %s c %s" % (tuple(_n(v) for v in (
                           cx + r, cy, cx + r, cy + k, cx + k, cy + r, cx, cy + r,
                           cx - k, cy + r, cx - r, cy + k, cx - r, cy,
                           cx - r, cy - k, cx - k, cy - r, cx, cy - r,
                           cx + k, cy - r, cx + r, cy - k, cx + r, cy)) + (op,)))
            ops.append("Q")
        elif tag == "text":
            s = "".join(el.itertext())
            size = float(el.get("font-size", base_size))
            bold = el.get("font-weight") == "bold"
            a, b, c, d = 1.0, 0.0, 0.0, 1.0
            e, f = float(el.get("x", "0")), float(el.get("y", "0"))
            tr = el.get("transform")
            if tr:
                m = re.match(r"translate\(\s*([-\d.]+)[ ,]+([-\d.]+)\s*\)\s*(?:rotate\(\s*([-\d.]+)\s*\))?", tr)
                if not m:
                    raise ValueError(f"unsupported transform {tr!r}")
                e, f = e + float(m.group(1)), f + float(m.group(2))
                if m.group(3):
                    th = math.radians(float(m.group(3)))
                    a, b, c, d = math.cos(th), math.sin(th), -math.sin(th), math.cos(th)
            anchor = el.get("text-anchor", "start")
            shift = {"start": 0.0, "middle": 0.5, "end": 1.0}[anchor] * text_width(s, size, bold)
            e, f = e - a * shift, f - b * shift
            col = fill if el.get("fill") is not None else (0.0, 0.0, 0.0)
            ops.append("BT %s %s %s rg /%s %s Tf %s %s %s %s %s %s Tm %s Tj ET"
                       % (*(_n(v) for v in col), "F2" if bold else "F1", _n(size),
                          _n(a), _n(b), _n(-c), _n(-d), _n(e), _n(f),
                          _pdf_str(s).decode("latin-1")))
    content = "\n".join(ops).encode("latin-1")
    gs = " ".join("/%s << /Type /ExtGState /ca %s >>" % (name, _n(alpha))
                  for alpha, name in sorted(page.alphas.items(), key=lambda kv: kv[1]))
    objects = [
        b"<< /Type /Catalog /Pages 2 0 R >>",
        b"<< /Type /Pages /Kids [3 0 R] /Count 1 >>",
        ("<< /Type /Page /Parent 2 0 R /MediaBox [0 0 %s %s] /Contents 4 0 R /Resources "
         "<< /Font << /F1 5 0 R /F2 6 0 R >> /ExtGState << %s >> >> >>" % (_n(W), _n(H), gs)).encode(),
        b"<< /Length %d >>\nstream\n" % len(content) + content + b"\nendstream",
        b"<< /Type /Font /Subtype /Type1 /BaseFont /Helvetica /Encoding /WinAnsiEncoding >>",
        b"<< /Type /Font /Subtype /Type1 /BaseFont /Helvetica-Bold /Encoding /WinAnsiEncoding >>",
    ]
    out = bytearray(b"%PDF-1.4\n%\xe2\xe3\xcf\xd3\n")
    offsets = []
    for i, body in enumerate(objects, 1):
        offsets.append(len(out))
        out += b"%d 0 obj\n" % i + body + b"\nendobj\n"
    xref = len(out)
    out += b"xref\n0 %d\n0000000000 65535 f \n" % (len(objects) + 1)
    for off in offsets:
        out += b"%010d 00000 n \n" % off
    out += b"trailer\n<< /Size %d /Root 1 0 R >>\nstartxref\n%d\n%%%%EOF\n" % (len(objects) + 1, xref)
    return bytes(out)
