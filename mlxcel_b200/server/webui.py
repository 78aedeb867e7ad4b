"""A single-page chat UI served at ``/`` (and ``/ui``): streams from ``/v1/chat/completions``.

The reference ships a React SPA embedded in the server binary (webui/, src/server/webui/*); this is
the same idea at the smallest useful size — one static HTML document with no build step and no
external assets, so it works on an air-gapped box.
"""

INDEX_HTML = """<!doctype html>
<html lang="en"><head><meta charset="utf-8"><title>mlxcel_b200</title>
<meta name="viewport" content="width=device-width, initial-scale=1">
<style>
 body{font:15px/1.45 system-ui,sans-serif;margin:0;display:flex;flex-direction:column;height:100vh;background:#111;color:#eee}
 header{padding:.6rem 1rem;background:#1b1b1b;border-bottom:1px solid #333;display:flex;gap:1rem;align-items:center}
 header b{flex:1} header span{color:#8a8;font-size:12px}
 #log{flex:1;overflow:auto;padding:1rem;max-width:60rem;width:100%;margin:0 auto;box-sizing:border-box}
 .m{white-space:pre-wrap;margin:.4rem 0;padding:.6rem .8rem;border-radius:.5rem}
 .user{background:#243447}.assistant{background:#1e1e1e;border:1px solid #333}
 form{display:flex;gap:.5rem;padding:.8rem;max-width:60rem;width:100%;margin:0 auto;box-sizing:border-box}
 textarea{flex:1;resize:none;height:3.2rem;background:#1b1b1b;color:#eee;border:1px solid #444;border-radius:.4rem;padding:.5rem}
 button{background:#2d6cdf;color:#fff;border:0;border-radius:.4rem;padding:0 1.2rem;cursor:pointer}
 input{width:5rem;background:#1b1b1b;color:#eee;border:1px solid #444;border-radius:.3rem;padding:.2rem}
</style></head><body>
<header><b>mlxcel_b200</b><label>max tokens <input id="mt" type="number" value="512"></label>
<label>temperature <input id="tp" type="number" step="0.1" value="0.7"></label><span id="st"></span></header>
<div id="log"></div>
<form id="f"><textarea id="q" placeholder="Message (Enter to send, Shift+Enter for a new line)"></textarea><button>Send</button></form>
<script>
const log=document.getElementById('log'),q=document.getElementById('q'),st=document.getElementById('st');
const msgs=[];
function add(role,text){const d=document.createElement('div');d.className='m '+role;d.textContent=text;log.appendChild(d);log.scrollTop=log.scrollHeight;return d}
fetch('/props').then(r=>r.json()).then(p=>{st.textContent=(p.model_alias||p.model_path||'')}).catch(()=>{});
q.addEventListener('keydown',e=>{if(e.key==='Enter'&&!e.shiftKey){e.preventDefault();document.getElementById('f').requestSubmit()}});
document.getElementById('f').addEventListener('submit',async e=>{
  e.preventDefault();const text=q.value.trim();if(!text)return;q.value='';
  msgs.push({role:'user',content:text});add('user',text);const out=add('assistant','');
  const t0=performance.now();let n=0,acc='';
  const r=await fetch('/v1/chat/completions',{method:'POST',headers:{'Content-Type':'application/json'},
    body:JSON.stringify({messages:msgs,stream:true,max_tokens:+document.getElementById('mt').value,temperature:+document.getElementById('tp').value})});
  const rd=r.body.getReader(),dec=new TextDecoder();let buf='';
  for(;;){const {done,value}=await rd.read();if(done)break;buf+=dec.decode(value,{stream:true});
    let i;while((i=buf.indexOf('\\n\\n'))>=0){const line=buf.slice(0,i);buf=buf.slice(i+2);
      if(!line.startsWith('data:'))continue;const d=line.slice(5).trim();if(d==='[DONE]')continue;
      try{const c=JSON.parse(d).choices[0].delta.content;if(c){acc+=c;n++;out.textContent=acc;log.scrollTop=log.scrollHeight}}catch(_){}}}
  msgs.push({role:'assistant',content:acc});st.textContent=n+' chunks, '+((performance.now()-t0)/1000).toFixed(1)+' s';
});
</script></body></html>
"""
