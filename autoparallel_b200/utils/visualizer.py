"""Self-contained HTML report of a solved plan.

``generate_visualization_html(optimizer.get_json(), trace=...)`` returns one HTML file (no external
assets, the plan and the trace are embedded as JSON) with six views behind tabs:

* **Overview** - mesh, cost totals, ILP size, planning timings, constraints, collective counts;
* **Modules** - a zoomable treemap of the module hierarchy (area = compute + communication time of
  the nodes traced inside a module, colour = share of communication) next to a collapsible module
  tree with the same totals;
* **Parameters** - the parameter tree by fully qualified name with placement, global shape, local
  shard size and the bytes each rank holds, folded per sub-module;
* **Hotspots** - the most expensive redistributions (producer, consumer, placement change);
* **Nodes** - every graph node with phase colouring and a text filter;
* **Timeline** - the simulated step (``utils.trace_sim.create_execution_trace``) drawn as compute
  and communication lanes, with the trace downloadable as Chrome-trace JSON for ui.perfetto.dev.

Reference: autoparallel/visualizer/build_display_from_json.py (module tree, treemap, parameter tree,
hotspot table, Perfetto tab: :1258-1739, entry point :2887).
"""
from __future__ import annotations

import html
import json
import math
from collections import defaultdict
from typing import Optional

_DTYPE_BYTES = {"torch.float32": 4, "torch.bfloat16": 2, "torch.float16": 2, "torch.float64": 8, "torch.int64": 8, "torch.int32": 4,
                "torch.bool": 1, "torch.uint8": 1, "torch.int8": 1, "torch.complex64": 8}


# ------------------------------------------------------------------------------------------ data shaping
def module_tree(nodes) -> dict:
    """Nested totals by module path: {"name", "compute", "comm", "n", "children": [...]}."""
    def new(name):
        return {"name": name, "compute": 0.0, "comm": 0.0, "n": 0, "children": {}}

    root = new("model")
    for n in nodes:
        path = [p for p in (n.get("module_path") or "").split(".") if p]
        comm = sum(e["comm_us"] for e in n["edges"])
        cur = root
        for p in [None] + path:
            if p is not None:
                cur = cur["children"].setdefault(p, new(p))
            cur["compute"] += n["compute_us"]
            cur["comm"] += comm
            cur["n"] += 1

    def freeze(t):
        kids = sorted((freeze(c) for c in t["children"].values()), key=lambda c: -(c["compute"] + c["comm"]))
        return {"name": t["name"], "compute": round(t["compute"], 2), "comm": round(t["comm"], 2), "n": t["n"], "children": kids}

    return freeze(root)


def _shard_factor(placement: str, mesh_shape) -> int:
    """How many ways a tensor is split by a placement string such as ``S(0)R`` or ``(S(0), S(1))``."""
    f, i, dim = 1, 0, 0
    toks = []
    while i < len(placement):
        c = placement[i]
        if c in "SRP":
            toks.append(c)
        i += 1
    for c, m in zip(toks, mesh_shape):
        if c == "S":
            f *= int(m)
        dim += 1
    return max(f, 1)


def parameter_tree(nodes, mesh_shape) -> dict:
    """Parameters nested by fqn: leaves carry placement, shape, dtype, local bytes; inner nodes the sums."""
    root = {"name": "parameters", "children": {}, "bytes": 0, "local_bytes": 0, "count": 0}
    for n in nodes:
        kind = n.get("kind")
        if not kind or kind[0] != "param":
            continue
        fqn = str(kind[1])
        numel = math.prod(n["shape"]) if n.get("shape") else 0
        nbytes = numel * _DTYPE_BYTES.get(n.get("dtype"), 4)
        local = nbytes // _shard_factor(n["placement"], mesh_shape)
        cur = root
        parts = fqn.split(".")
        for i, p in enumerate(parts):
            cur["bytes"] += nbytes
            cur["local_bytes"] += local
            cur["count"] += 1
            cur = cur["children"].setdefault(p, {"name": p, "children": {}, "bytes": 0, "local_bytes": 0, "count": 0})
        cur.update(bytes=nbytes, local_bytes=local, count=1, placement=n["placement"], shape=n["shape"], dtype=n["dtype"], fqn=fqn)

    def freeze(t):
        out = {k: v for k, v in t.items() if k != "children"}
        out["children"] = [freeze(c) for c in t["children"].values()]
        return out

    return freeze(root)


def _fmt_bytes(b: float) -> str:
    for unit in ("B", "KiB", "MiB", "GiB", "TiB"):
        if abs(b) < 1024 or unit == "TiB":
            return f"{b:.1f} {unit}" if unit != "B" else f"{int(b)} B"
        b /= 1024
    return f"{b:.1f} TiB"


def _render_module_tree(t, depth=0) -> str:
    label = (f"<b>{html.escape(t['name'])}</b> <span class=dim>{t['n']} nodes</span> "
             f"<span class=c>{t['compute']:.0f} µs compute</span> <span class=m>{t['comm']:.0f} µs comm</span>")
    kids = "".join(_render_module_tree(c, depth + 1) for c in t["children"])
    if not kids:
        return f"<div class=leaf style='margin-left:{depth * 14}px'>{label}</div>"
    return f"<details {'open' if depth < 1 else ''} style='margin-left:{depth * 14}px'><summary>{label}</summary>{kids}</details>"


def _render_param_tree(t, depth=0) -> str:
    if not t["children"]:
        return (f"<div class=leaf style='margin-left:{depth * 14}px'><b>{html.escape(t['name'])}</b> "
                f"<span class=pl>{html.escape(t.get('placement', ''))}</span> {t.get('shape')} <span class=dim>{t.get('dtype', '')}</span> "
                f"<span class=c>{_fmt_bytes(t['local_bytes'])} per rank</span> <span class=dim>of {_fmt_bytes(t['bytes'])}</span></div>")
    label = (f"<b>{html.escape(t['name'])}</b> <span class=dim>{t['count']} tensors</span> "
             f"<span class=c>{_fmt_bytes(t['local_bytes'])} per rank</span> <span class=dim>of {_fmt_bytes(t['bytes'])}</span>")
    kids = "".join(_render_param_tree(c, depth + 1) for c in t["children"])
    return f"<details {'open' if depth < 2 else ''} style='margin-left:{depth * 14}px'><summary>{label}</summary>{kids}</details>"


_CSS = """
body{font:13px system-ui,sans-serif;margin:0} header{padding:10px 16px;background:#1f2937;color:#fff}
header h1{font-size:16px;margin:0 0 4px 0} nav{display:flex;gap:2px;background:#e5e7eb;padding:0 12px}
nav button{border:0;background:none;padding:8px 14px;cursor:pointer;font:inherit} nav button.on{background:#fff;font-weight:600}
section{display:none;padding:14px 16px} section.on{display:block}
table{border-collapse:collapse} td,th{border:1px solid #ddd;padding:2px 6px;text-align:left}
tr.backward{background:#fff5f0} tr.forward{background:#f3f8ff} .dim{color:#888} .c{color:#06c} .m{color:#c30} .pl{color:#070;font-family:monospace}
details{margin:2px 0} input{margin:6px 0;width:320px} .cols{display:flex;gap:18px;align-items:flex-start}
#treemap{position:relative;width:880px;height:520px;border:1px solid #999;overflow:hidden;flex:none}
#treemap div{position:absolute;box-sizing:border-box;border:1px solid #fff;overflow:hidden;font-size:11px;padding:1px 3px;cursor:pointer;color:#111}
#crumbs{margin-bottom:6px} #crumbs a{cursor:pointer;color:#06c} canvas{border:1px solid #999}
.kv td:first-child{font-weight:600}
"""

_JS = r"""
function show(id){for(const s of document.querySelectorAll('section'))s.classList.toggle('on',s.id===id);
 for(const b of document.querySelectorAll('nav button'))b.classList.toggle('on',b.dataset.t===id);
 if(id==='modules')drawTreemap(zoomPath); if(id==='timeline')drawTimeline();}
function flt(){const q=document.getElementById('f').value.toLowerCase();
 for(const r of document.querySelectorAll('#t tr')){if(!r.querySelector('td'))continue;r.style.display=r.textContent.toLowerCase().includes(q)?'':'none';}}
// ---- squarified treemap of the module tree
let zoomPath=[];
function total(n){return n.compute+n.comm;}
function squarify(items,x,y,w,h,out){ // items sorted by value, descending
 let rest=items.slice(), sum=rest.reduce((a,b)=>a+b.v,0);
 while(rest.length){ const horiz=w>=h, side=horiz?h:w; let row=[], rowSum=0, best=Infinity, i=0;
  for(;i<rest.length;i++){ const r=row.concat([rest[i]]), s=rowSum+rest[i].v; const thick=s/sum*(horiz?w:h);
   let worst=0; for(const it of r){const len=it.v/s*side; worst=Math.max(worst,Math.max(thick/len,len/thick));}
   if(worst>best)break; best=worst; row=r; rowSum=s; }
  const thick=rowSum/sum*(horiz?w:h); let off=0;
  for(const it of row){const len=it.v/rowSum*side; out.push(horiz?{n:it.n,x:x,y:y+off,w:thick,h:len}:{n:it.n,x:x+off,y:y,w:len,h:thick}); off+=len;}
  if(horiz){x+=thick;w-=thick;}else{y+=thick;h-=thick;} rest=rest.slice(row.length); sum-=rowSum; } }
function nodeAt(path){let n=DATA.modules; for(const p of path){n=n.children.find(c=>c.name===p);} return n;}
function drawTreemap(path){ zoomPath=path; const el=document.getElementById('treemap'); el.innerHTML=''; const node=nodeAt(path);
 const kids=(node.children.length?node.children:[node]).filter(c=>total(c)>0).map(c=>({n:c,v:total(c)})); const rects=[];
 squarify(kids,0,0,el.clientWidth,el.clientHeight,rects);
 for(const r of rects){const d=document.createElement('div'); const share=r.n.comm/Math.max(total(r.n),1e-9);
  d.style.cssText=`left:${r.x}px;top:${r.y}px;width:${r.w}px;height:${r.h}px;background:hsl(${210-190*share},70%,${78-18*share}%)`;
  d.title=`${r.n.name}: ${r.n.compute.toFixed(0)} µs compute, ${r.n.comm.toFixed(0)} µs communication, ${r.n.n} nodes`;
  d.textContent=`${r.n.name} ${total(r.n).toFixed(0)} µs`; if(r.n.children.length)d.onclick=()=>drawTreemap(path.concat([r.n.name])); el.appendChild(d);}
 const c=document.getElementById('crumbs'); c.innerHTML='';
 ['model'].concat(path).forEach((p,i)=>{const a=document.createElement('a');a.textContent=p;a.onclick=()=>drawTreemap(path.slice(0,i));c.appendChild(a);
  if(i<path.length)c.appendChild(document.createTextNode(' › '));}); }
// ---- timeline of the simulated step
function drawTimeline(){ const cv=document.getElementById('tl'); if(!DATA.trace){return;} const ev=DATA.trace.traceEvents.filter(e=>e.ph==='X');
 const lanes=[...new Set(ev.map(e=>e.pid+':'+e.tid))].sort(); const t0=Math.min(...ev.map(e=>e.ts)), t1=Math.max(...ev.map(e=>e.ts+e.dur));
 const W=cv.width, laneH=34; cv.height=lanes.length*laneH+24; const g=cv.getContext('2d'); g.clearRect(0,0,W,cv.height); g.font='11px system-ui';
 lanes.forEach((l,i)=>{g.fillStyle='#f3f4f6';g.fillRect(0,i*laneH+20,W,laneH-4);g.fillStyle='#111';g.fillText(laneName(l),4,i*laneH+16);});
 for(const e of ev){const i=lanes.indexOf(e.pid+':'+e.tid); const x=(e.ts-t0)/(t1-t0)*W, w=Math.max(e.dur/(t1-t0)*W,0.5);
  g.fillStyle=/all_gather|reduce_scatter|all_reduce|all_to_all|comm/.test(e.name)?'#dc2626':(/mm|gemm|attention/.test(e.name)?'#2563eb':'#6b7280');
  g.fillRect(x,i*laneH+22,w,laneH-8);} g.fillStyle='#111'; g.fillText(((t1-t0)/1000).toFixed(2)+' ms simulated',W-130,12); }
function laneName(l){const m=(DATA.trace.traceEvents||[]).find(e=>e.ph==='M'&&e.name==='thread_name'&&(e.pid+':'+e.tid)===l);return m?m.args.name:l;}
function downloadTrace(){const b=new Blob([JSON.stringify(DATA.trace)],{type:'application/json'});const a=document.createElement('a');
 a.href=URL.createObjectURL(b);a.download='simulated_step.trace.json';a.click();}
"""


def generate_visualization_html(plan: dict, title: str = "autoparallel_b200 plan", trace: Optional[dict] = None) -> str:
    """``plan``: ``ShardingOptimizer.get_json()``; ``trace``: Chrome-trace dict of the simulated step (optional)."""
    nodes = plan["nodes"]
    s = plan["summary"]
    mesh = plan["mesh"]
    modules = module_tree(nodes)
    ptree = parameter_tree(nodes, mesh["shape"])
    edges = sorted(((e["comm_us"], n["name"], e) for n in nodes for e in n["edges"] if e["comm_us"] > 0), key=lambda x: -x[0])[:60]
    rows = []
    for n in nodes:
        comm = sum(e["comm_us"] for e in n["edges"])
        redis = "; ".join(f"{e['from']}: {e['src_placement']}→{e['dst_placement']} ({e['comm_us']:.1f})" for e in n["edges"] if e["comm_us"] > 0)
        rows.append(
            f"<tr class={n['phase']}><td>{html.escape(n['name'])}</td><td>{html.escape(n['target'][:48])}</td><td>{n['phase'][:3]}</td>"
            f"<td class=pl>{html.escape(n['placement'])}</td><td>{n['shape']}</td><td>{n['compute_us']:.1f}</td><td>{comm:.1f}</td>"
            f"<td>{html.escape(redis)}</td><td>{html.escape(n.get('module_path') or '')}</td></tr>")
    hot = "".join(f"<tr><td>{c:.1f}</td><td>{html.escape(nm)}</td><td>{html.escape(e['from'])}</td><td class=pl>{e['src_placement']} → {e['dst_placement']}</td></tr>"
                  for c, nm, e in edges)
    by_change = defaultdict(float)
    for c, _, e in edges:
        by_change[f"{e['src_placement']} → {e['dst_placement']}"] += c
    changes = "".join(f"<tr><td class=pl>{html.escape(k)}</td><td>{v:.1f}</td></tr>" for k, v in sorted(by_change.items(), key=lambda kv: -kv[1]))
    overview = "".join(f"<tr><td>{html.escape(str(k))}</td><td>{html.escape(str(v))}</td></tr>" for k, v in (
        ("mesh", f"{mesh['shape']} {mesh['dim_names']} on {mesh['device_type']}"), ("nodes", s["num_nodes"]),
        ("compute (µs, sum over nodes)", f"{s['compute_us']:.0f}"), ("communication (µs)", f"{s['comm_us']:.0f}"),
        ("objective", s["objective"]), ("ILP", s["ilp"]), ("planning timings (s)", s["timings_s"]),
        ("constraints", json.dumps(s["constraints"])), ("parameters per rank", f"{_fmt_bytes(ptree['local_bytes'])} of {_fmt_bytes(ptree['bytes'])}"),
    ))
    timeline = ("<p><button onclick='downloadTrace()'>download Chrome-trace JSON</button> (open in ui.perfetto.dev) · red: collectives, "
                "blue: GEMM / attention, grey: other</p><canvas id=tl width=1200 height=120></canvas>") if trace else \
        "<p class=dim>no simulated trace was passed (generate_visualization_html(plan, trace=create_execution_trace(...)))</p>"
    data = {"plan": plan, "modules": modules, "parameters": ptree, "trace": trace}
    return f"""<!doctype html><html><head><meta charset=utf-8><title>{html.escape(title)}</title><style>{_CSS}</style></head><body>
<header><h1>{html.escape(title)}</h1>mesh {mesh['shape']} {mesh['dim_names']} · {s['num_nodes']} nodes · compute {s['compute_us']:.0f} µs ·
communication {s['comm_us']:.0f} µs</header>
<nav>{''.join(f"<button data-t={t} onclick=show('{t}') class={'on' if i == 0 else ''}>{lbl}</button>" for i, (t, lbl) in enumerate(
        (('overview', 'Overview'), ('modules', 'Modules'), ('parameters', 'Parameters'), ('hotspots', 'Hotspots'), ('nodes', 'Nodes'), ('timeline', 'Timeline'))))}</nav>
<section id=overview class=on><table class=kv>{overview}</table></section>
<section id=modules><div id=crumbs></div><div class=cols><div id=treemap></div><div>{_render_module_tree(modules)}</div></div>
<p class=dim>area: compute + communication time of the nodes traced inside a module; colour: blue = compute, red = communication; click to zoom</p></section>
<section id=parameters>{_render_param_tree(ptree)}</section>
<section id=hotspots><div class=cols><div><h3>Most expensive redistributions</h3><table><tr><th>µs</th><th>consumer</th><th>producer</th><th>change</th></tr>{hot}</table></div>
<div><h3>By placement change</h3><table><tr><th>change</th><th>µs</th></tr>{changes}</table></div></div></section>
<section id=nodes><input id=f placeholder="filter (name, op, placement, module)…" oninput="flt()">
<table id=t><tr><th>node</th><th>op</th><th>ph</th><th>placement</th><th>shape</th><th>compute µs</th><th>comm µs</th><th>redistributions</th><th>module</th></tr>
{''.join(rows)}</table></section>
<section id=timeline>{timeline}</section>
<script>const DATA={json.dumps(data)};{_JS}</script>
</body></html>"""


def write_report(path: str, optimizer, lowered_gm=None, mesh=None, title: str = "autoparallel_b200 plan") -> str:
    """Plan JSON + (when the lowered graph is given) the simulated step trace -> one HTML file at ``path``."""
    trace = None
    if lowered_gm is not None and mesh is not None:
        from .trace_sim import create_execution_trace

        trace = create_execution_trace(lowered_gm, mesh)
    doc = generate_visualization_html(optimizer.get_json(), title=title, trace=trace)
    with open(path, "w") as f:
        f.write(doc)
    return path
