"""Self-contained HTML report of a solved plan.

``generate_visualization_html(optimizer.get_json())`` returns one HTML string (no external assets)
with: a summary header (mesh, costs, ILP size), a collapsible module tree with per-module compute /
communication totals, a parameter table (placement, shard ratio), a hotspot table (the most
expensive redistributions), and the full node table with forward/backward phase colouring and
filtering.  The plan JSON is embedded, so the file can be post-processed.  Reference:
autoparallel/visualizer/build_display_from_json.py (module tree, treemap, parameter tree, hotspot
table; ~3.4 kLoC of HTML-in-Python).
"""
from __future__ import annotations

import html
import json
from collections import defaultdict


def _module_tree(nodes):
    tree = lambda: {"compute": 0.0, "comm": 0.0, "n": 0, "children": defaultdict(tree)}  # noqa: E731
    root = tree()
    for n in nodes:
        path = [p for p in (n.get("module_path") or "").split(".") if p]
        comm = sum(e["comm_us"] for e in n["edges"])
        cur = root
        cur["compute"] += n["compute_us"]
        cur["comm"] += comm
        cur["n"] += 1
        for p in path:
            cur = cur["children"][p]
            cur["compute"] += n["compute_us"]
            cur["comm"] += comm
            cur["n"] += 1
    return root


def _render_tree(name, t, depth=0):
    kids = "".join(_render_tree(k, v, depth + 1) for k, v in sorted(t["children"].items(), key=lambda kv: -kv[1]["compute"] - kv[1]["comm"]))
    label = (f"<b>{html.escape(name)}</b> <span class=dim>{t['n']} nodes</span> "
             f"<span class=c>{t['compute']:.0f} µs compute</span> <span class=m>{t['comm']:.0f} µs comm</span>")
    if not kids:
        return f"<div class=leaf style='margin-left:{depth * 14}px'>{label}</div>"
    return f"<details {'open' if depth < 1 else ''} style='margin-left:{depth * 14}px'><summary>{label}</summary>{kids}</details>"


def generate_visualization_html(plan: dict, title: str = "autoparallel_b200 plan") -> str:
    nodes = plan["nodes"]
    s = plan["summary"]
    mesh = plan["mesh"]
    params = [n for n in nodes if n.get("kind") and n["kind"][0] == "param"]
    edges = sorted(((e["comm_us"], n["name"], e) for n in nodes for e in n["edges"] if e["comm_us"] > 0), key=lambda x: -x[0])[:40]
    rows = []
    for n in nodes:
        comm = sum(e["comm_us"] for e in n["edges"])
        redis = "; ".join(f"{e['from']}: {e['src_placement']}→{e['dst_placement']} ({e['comm_us']:.1f})" for e in n["edges"] if e["comm_us"] > 0)
        rows.append(
            f"<tr class={n['phase']}><td>{html.escape(n['name'])}</td><td>{html.escape(n['target'][:48])}</td><td>{n['phase'][:3]}</td>"
            f"<td>{html.escape(n['placement'])}</td><td>{n['shape']}</td><td>{n['compute_us']:.1f}</td><td>{comm:.1f}</td>"
            f"<td>{html.escape(redis)}</td><td>{html.escape(n.get('module_path') or '')}</td></tr>")
    prow = "".join(f"<tr><td>{html.escape(str(p['kind'][1]))}</td><td>{p['placement']}</td><td>{p['shape']}</td><td>{p['dtype']}</td></tr>" for p in params)
    hot = "".join(f"<tr><td>{c:.1f}</td><td>{html.escape(nm)}</td><td>{html.escape(e['from'])}</td><td>{e['src_placement']} → {e['dst_placement']}</td></tr>"
                  for c, nm, e in edges)
    return f"""<!doctype html><html><head><meta charset=utf-8><title>{html.escape(title)}</title><style>
body{{font:13px system-ui,sans-serif;margin:16px}} table{{border-collapse:collapse}} td,th{{border:1px solid #ddd;padding:2px 6px}}
tr.backward{{background:#fff5f0}} tr.forward{{background:#f3f8ff}} .dim{{color:#888}} .c{{color:#06c}} .m{{color:#c30}}
details{{margin:2px 0}} input{{margin:6px 0;width:320px}} h2{{margin-top:22px}}</style></head><body>
<h1>{html.escape(title)}</h1>
<p>mesh {mesh['shape']} {mesh['dim_names']} on {mesh['device_type']} · {s['num_nodes']} nodes · compute {s['compute_us']:.0f} µs ·
communication {s['comm_us']:.0f} µs · objective {s['objective']} · ILP {s['ilp']} · timings {s['timings_s']}</p>
<p>constraints: {html.escape(json.dumps(s['constraints']))}</p>
<h2>Module tree</h2>{_render_tree('model', _module_tree(nodes))}
<h2>Parameters</h2><table><tr><th>fqn</th><th>placement</th><th>shape</th><th>dtype</th></tr>{prow}</table>
<h2>Most expensive redistributions</h2><table><tr><th>µs</th><th>consumer</th><th>producer</th><th>change</th></tr>{hot}</table>
<h2>Nodes</h2><input id=f placeholder="filter (name, op, placement, module)…" oninput="flt()">
<table id=t><tr><th>node</th><th>op</th><th>ph</th><th>placement</th><th>shape</th><th>compute µs</th><th>comm µs</th><th>redistributions</th><th>module</th></tr>
{''.join(rows)}</table>
<script>const plan={json.dumps(plan)};
function flt(){{const q=document.getElementById('f').value.toLowerCase();for(const r of document.querySelectorAll('#t tr')){{if(!r.querySelector('td'))continue;r.style.display=r.textContent.toLowerCase().includes(q)?'':'none';}}}}</script>
</body></html>"""
