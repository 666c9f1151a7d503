"""HTML view of a fused graph (`plowc viz`; reference: crates/nn-graph/src/viz/)."""
from __future__ import annotations

import html


def to_html(g) -> str:
    rows = []
    for k, n in enumerate(g.nodes):
        ins = ", ".join(html.escape(str(i)) for i in n.inputs if i is not None)
        outs = ", ".join(html.escape(o) for o in n.outputs)
        cls = "fused" if n.site else "prim"
        rows.append(f"<tr class='{cls}'><td>{k}</td><td>{n.layer}</td><td><b>{html.escape(n.op)}</b></td>"
                    f"<td>{html.escape(n.site)}</td><td>{ins}</td><td>{outs}</td></tr>")
    return ("<html><head><style>body{font-family:monospace}td{padding:2px 8px;border-bottom:1px solid #ddd}"
            ".fused{background:#e8f4e8}</style></head><body><h3>" + html.escape(g.spec.model_type) +
            f" — {len(g.nodes)} nodes</h3><table><tr><th>#</th><th>layer</th><th>op</th><th>site</th><th>inputs</th>"
            "<th>outputs</th></tr>" + "".join(rows) + "</table></body></html>")
