"""The dashboard: one static page served at ``/`` that talks to the REST API with ``fetch`` and to
the metrics stream with a WebSocket.  Pages: overview, training (live loss chart), models,
datasets, inference, hub, notebooks, system, admin — the page list of the reference's Leptos
single-page application (crates/axonml-dashboard/src/pages), without a build step or WASM."""

PAGE = r"""<!doctype html>
<html lang="en"><head><meta charset="utf-8"><title>AxonML</title>
<meta name="viewport" content="width=device-width, initial-scale=1">
<style>
:root{--bg:#0f1419;--panel:#1a212b;--line:#2b3644;--fg:#d8dee9;--dim:#8a97a8;--acc:#14b8a6;--bad:#ef4444}
*{box-sizing:border-box}body{margin:0;font:14px/1.45 system-ui,sans-serif;background:var(--bg);color:var(--fg);display:flex;min-height:100vh}
nav{width:190px;background:var(--panel);border-right:1px solid var(--line);padding:14px 0;flex-shrink:0}
nav h1{font-size:17px;margin:0 16px 14px;color:var(--acc)}nav a{display:block;padding:8px 16px;color:var(--fg);text-decoration:none;cursor:pointer}
nav a.on,nav a:hover{background:#232d3a;color:var(--acc)}main{flex:1;padding:22px;overflow:auto}
h2{margin:0 0 14px;font-size:19px}.cards{display:grid;grid-template-columns:repeat(auto-fill,minmax(170px,1fr));gap:12px;margin-bottom:18px}
.card{background:var(--panel);border:1px solid var(--line);border-radius:8px;padding:12px}.card b{display:block;font-size:22px;color:var(--acc)}
table{width:100%;border-collapse:collapse;background:var(--panel);border:1px solid var(--line);border-radius:8px}
th,td{text-align:left;padding:7px 10px;border-bottom:1px solid var(--line)}th{color:var(--dim);font-weight:500}
input,select,button,textarea{font:inherit;background:#111821;color:var(--fg);border:1px solid var(--line);border-radius:6px;padding:6px 9px}
button{background:var(--acc);color:#062925;border:0;cursor:pointer;font-weight:600}button.ghost{background:transparent;color:var(--fg);border:1px solid var(--line)}
form.row{display:flex;gap:8px;flex-wrap:wrap;margin:0 0 14px}.err{color:var(--bad)}.dim{color:var(--dim)}
canvas{background:var(--panel);border:1px solid var(--line);border-radius:8px;width:100%;height:240px}
pre{background:#0b1016;border:1px solid var(--line);border-radius:6px;padding:8px;overflow:auto;margin:6px 0}
#login{max-width:340px;margin:12vh auto;background:var(--panel);padding:22px;border-radius:10px;border:1px solid var(--line)}
#login input{width:100%;margin-bottom:10px}
</style></head><body>
<nav id="nav" hidden><h1>AxonML</h1>
<a data-p="overview">Overview</a><a data-p="training">Training</a><a data-p="models">Models</a><a data-p="datasets">Datasets</a>
<a data-p="inference">Inference</a><a data-p="hub">Hub</a><a data-p="notebooks">Notebooks</a><a data-p="system">System</a>
<a data-p="admin">Admin</a><a id="logout">Log out</a></nav>
<main id="main"></main>
<script>
const $=s=>document.querySelector(s), main=$('#main');
let token=localStorage.getItem('axonml_token')||'', socket=null;
const esc=s=>String(s??'').replace(/[&<>"]/g,c=>({'&':'&amp;','<':'&lt;','>':'&gt;','"':'&quot;'}[c]));
async function api(method,path,body){const r=await fetch(path,{method,headers:{'Content-Type':'application/json',...(token?{Authorization:'Bearer '+token}:{})},body:body?JSON.stringify(body):undefined});
 const t=await r.text();let j;try{j=JSON.parse(t)}catch(e){j=t}if(r.status===401&&path!=='/api/auth/login'){token='';showLogin();throw new Error('signed out')}
 if(!r.ok)throw new Error(j.error||r.statusText);return j}
function table(rows,cols,actions){if(!rows.length)return '<p class="dim">nothing here yet</p>';
 return '<table><tr>'+cols.map(c=>'<th>'+esc(c)+'</th>').join('')+(actions?'<th></th>':'')+'</tr>'+rows.map(r=>'<tr>'+cols.map(c=>'<td>'+esc(typeof r[c]==='object'&&r[c]?JSON.stringify(r[c]):r[c])+'</td>').join('')+(actions?'<td>'+actions(r)+'</td>':'')+'</tr>').join('')+'</table>'}
function showLogin(msg){$('#nav').hidden=true;main.innerHTML=`<div id="login"><h2>Sign in</h2><p class="err">${esc(msg||'')}</p>
 <input id="em" placeholder="e-mail"><input id="pw" type="password" placeholder="password"><input id="otp" placeholder="authenticator code (if enabled)">
 <button id="go">Sign in</button> <button class="ghost" id="reg">Register</button></div>`;
 $('#go').onclick=async()=>{try{let j=await api('POST','/api/auth/login',{email:$('#em').value,password:$('#pw').value});
  if(j.requires_mfa){j=await api('POST','/api/auth/mfa/totp/verify',{mfa_token:j.mfa_token,code:$('#otp').value})}
  token=j.access_token;localStorage.setItem('axonml_token',token);start()}catch(e){showLogin(e.message)}};
 $('#reg').onclick=async()=>{try{await api('POST','/api/auth/register',{email:$('#em').value,name:$('#em').value.split('@')[0],password:$('#pw').value});showLogin('registered: sign in')}catch(e){showLogin(e.message)}}}
const pages={
 async overview(){const [s,runs,models]=await Promise.all([api('GET','/api/system/info'),api('GET','/api/training/runs'),api('GET','/api/models')]);
  main.innerHTML=`<h2>Overview</h2><div class="cards"><div class="card"><b>${runs.length}</b>training runs</div><div class="card"><b>${runs.filter(r=>r.status==='running').length}</b>running</div>
  <div class="card"><b>${models.length}</b>models</div><div class="card"><b>${s.gpu_count}</b>GPUs</div><div class="card"><b>${s.cpu_count}</b>CPU cores</div></div>
  <h2>Recent runs</h2>${table(runs.slice(0,8),['name','model_type','status','started_at'])}`},
 async training(){const runs=await api('GET','/api/training/runs');
  main.innerHTML=`<h2>Training</h2><form class="row" id="f"><input name="name" placeholder="run name" required><select name="model_type"><option>mlp</option><option>lenet</option><option>simplecnn</option></select>
  <input name="epochs" type="number" value="2" style="width:80px" title="epochs"><input name="lr" value="0.001" style="width:90px" title="learning rate"><button>Start run</button></form>
  <canvas id="chart" width="900" height="240"></canvas><p id="live" class="dim">select a run to watch its loss</p>
  ${table(runs,['name','model_type','status','latest_metrics'],r=>`<button class="ghost" onclick="watch('${r.id}')">watch</button> <button class="ghost" onclick="stopRun('${r.id}')">stop</button>`)}`;
  $('#f').onsubmit=async e=>{e.preventDefault();const f=new FormData(e.target);const r=await api('POST','/api/training/runs',{name:f.get('name'),model_type:f.get('model_type'),config:{epochs:+f.get('epochs'),learning_rate:+f.get('lr'),steps_per_epoch:50}});await pages.training();watch(r.id)}},
 async models(){const m=await api('GET','/api/models');main.innerHTML=`<h2>Models</h2><form class="row" id="f"><input name="name" placeholder="model name" required><input name="description" placeholder="description"><button>Create</button></form>${table(m,['name','model_type','version_count','created_at'])}`;
  $('#f').onsubmit=async e=>{e.preventDefault();const f=new FormData(e.target);await api('POST','/api/models',{name:f.get('name'),description:f.get('description')});pages.models()}},
 async datasets(){const d=await api('GET','/api/datasets');const b=await api('GET','/api/builtin-datasets');main.innerHTML=`<h2>Datasets</h2>${table(d,['name','dataset_type','file_size','num_samples'])}<h2 style="margin-top:18px">Catalogue</h2>${table(b,['id','name','type','samples','classes'])}`},
 async inference(){const e=await api('GET','/api/inference/endpoints');const s=await api('GET','/api/status/inference');main.innerHTML=`<h2>Inference</h2><div class="cards"><div class="card"><b>${s.endpoints_running}</b>endpoints running</div><div class="card"><b>${s.llm?'yes':'no'}</b>LLM loaded</div></div>${table(e,['name','model_id','version','status','request_count'],r=>`<button class="ghost" onclick="ep('${r.id}','start')">start</button> <button class="ghost" onclick="ep('${r.id}','stop')">stop</button>`)}`},
 async hub(){const h=await api('GET','/api/hub/models');main.innerHTML=`<h2>Model hub</h2>${table(h,['name','architecture','category','parameters','size_mb','cached'])}`},
 async notebooks(){const n=await api('GET','/api/notebooks');main.innerHTML=`<h2>Notebooks</h2><form class="row" id="f"><input name="name" placeholder="notebook name" required><button>Create</button></form>${table(n,['name','status','created_at'],r=>`<button class="ghost" onclick="openNb('${r.id}')">open</button>`)}<div id="nb"></div>`;
  $('#f').onsubmit=async e=>{e.preventDefault();await api('POST','/api/notebooks',{name:new FormData(e.target).get('name')});pages.notebooks()}},
 async system(){const [s,m]=await Promise.all([api('GET','/api/system/info'),api('GET','/api/system/metrics')]);main.innerHTML=`<h2>System</h2><div class="cards"><div class="card"><b>${m.cpu_percent}%</b>CPU</div><div class="card"><b>${((m.memory_used_bytes||0)/2**30).toFixed(1)} GB</b>memory used</div><div class="card"><b>${esc(s.torch)}</b>torch</div><div class="card"><b>${esc(s.cuda)}</b>CUDA</div></div>${table(s.gpus,['id','name','memory_total','memory_used','utilization','temperature','power_w'])}`},
 async admin(){try{const [u,st]=await Promise.all([api('GET','/api/admin/users'),api('GET','/api/admin/stats')]);main.innerHTML=`<h2>Admin</h2><div class="cards">${Object.entries(st).filter(([k,v])=>typeof v==='number').map(([k,v])=>`<div class="card"><b>${v}</b>${esc(k)}</div>`).join('')}</div>${table(u,['email','name','role','mfa_enabled','last_login'])}`}catch(e){main.innerHTML='<h2>Admin</h2><p class="err">'+esc(e.message)+'</p>'}}};
window.stopRun=async id=>{await api('POST',`/api/training/runs/${id}/stop`);pages.training()};
window.ep=async(id,a)=>{await api('POST',`/api/inference/endpoints/${id}/${a}`);pages.inference()};
window.openNb=async id=>{const n=await api('GET','/api/notebooks/'+id);$('#nb').innerHTML='<h2 style="margin-top:18px">'+esc(n.name)+'</h2>'+n.cells.map(c=>`<div class="card" style="margin-bottom:8px"><span class="dim">${c.cell_type}</span>
 <textarea style="width:100%;min-height:70px" id="src_${c.id}">${esc(c.source)}</textarea>${c.cell_type==='code'?`<button onclick="runCell('${id}','${c.id}')">run</button>`:''}
 ${(c.outputs||[]).map(o=>'<pre>'+esc(o.text||((o.error_name||'')+': '+(o.error_value||'')))+'</pre>').join('')}</div>`).join('')+`<button class="ghost" onclick="addCell('${id}')">+ cell</button>`};
window.runCell=async(nb,c)=>{await api('PUT',`/api/notebooks/${nb}/cells/${c}`,{source:$('#src_'+c).value});await api('POST',`/api/notebooks/${nb}/cells/${c}/execute`);openNb(nb)};
window.addCell=async nb=>{await api('POST',`/api/notebooks/${nb}/cells`,{cell_type:'code',source:''});openNb(nb)};
window.watch=async id=>{if(socket)socket.close();const pts=(await api('GET',`/api/training/runs/${id}/metrics`)).map(m=>[m.step,m.loss]);draw(pts);
 socket=new WebSocket((location.protocol==='https:'?'wss://':'ws://')+location.host+`/api/training/runs/${id}/stream?token=${token}`);
 socket.onmessage=e=>{const m=JSON.parse(e.data);if(m.type==='metrics'){pts.push([m.data.step,m.data.loss]);draw(pts);$('#live').textContent=`step ${m.data.step}  loss ${(+m.data.loss).toFixed(4)}  accuracy ${m.data.accuracy!=null?(+m.data.accuracy).toFixed(3):'-'}`}else{$('#live').textContent='status: '+m.data.status}}};
function draw(pts){const c=$('#chart');if(!c)return;const g=c.getContext('2d');g.clearRect(0,0,c.width,c.height);pts=pts.filter(p=>p[1]!=null);if(pts.length<2)return;
 const xs=pts.map(p=>p[0]),ys=pts.map(p=>p[1]),x0=Math.min(...xs),x1=Math.max(...xs),y0=Math.min(...ys),y1=Math.max(...ys);
 g.strokeStyle='#14b8a6';g.lineWidth=2;g.beginPath();pts.forEach((p,i)=>{const x=20+(p[0]-x0)/(x1-x0||1)*(c.width-40),y=c.height-20-(p[1]-y0)/(y1-y0||1)*(c.height-40);i?g.lineTo(x,y):g.moveTo(x,y)});g.stroke();
 g.fillStyle='#8a97a8';g.fillText(y1.toFixed(3),4,14);g.fillText(y0.toFixed(3),4,c.height-6)}
function go(p){document.querySelectorAll('nav a').forEach(a=>a.classList.toggle('on',a.dataset.p===p));pages[p]().catch(e=>{if(e.message!=='signed out')main.innerHTML='<p class="err">'+esc(e.message)+'</p>'})}
function start(){$('#nav').hidden=false;go('overview')}
document.querySelectorAll('nav a[data-p]').forEach(a=>a.onclick=()=>go(a.dataset.p));
$('#logout').onclick=async()=>{try{await api('POST','/api/auth/logout')}catch(e){}token='';localStorage.removeItem('axonml_token');showLogin()};
token?start():showLogin();
</script></body></html>
"""
