"""Browser console of the server: one static page (HTML + a few lines of JavaScript, nothing to build) served at
``/`` and ``/console``.  It talks to the same process through the public routes only -- ``/health``, ``/v1/models``
and ``/v1/chat/completions`` with ``stream: true`` -- so whatever the console can do, any client can do.  The page is
served without a key (it holds no data); the key typed into it goes out as a bearer header with every call.

Reference: the plain-Python browser consoles of the reference (ninfer-gui.py, tools/gui/*.py: pages over
``ThreadingHTTPServer``, no graphics API anywhere).
"""
from __future__ import annotations

PAGE = """<!doctype html>
<html lang="en"><head><meta charset="utf-8"><title>ninfer-fusion-b200 console</title>
<meta name="viewport" content="width=device-width, initial-scale=1">
<style>
 body{font:14px/1.45 system-ui,sans-serif;margin:0;background:#111;color:#ddd;display:flex;flex-direction:column;height:100vh}
 header{padding:8px 12px;background:#1b1b1b;border-bottom:1px solid #333;display:flex;gap:10px;align-items:center;flex-wrap:wrap}
 header input,header select{background:#222;color:#ddd;border:1px solid #444;border-radius:4px;padding:4px 6px}
 #log{flex:1;overflow:auto;padding:12px}
 .msg{max-width:900px;margin:0 auto 10px;padding:8px 10px;border-radius:6px;white-space:pre-wrap;word-break:break-word}
 .user{background:#1e2a3a}.assistant{background:#1d1d1d;border:1px solid #2c2c2c}.think{color:#8a8a8a;font-style:italic}
 .err{background:#3a1e1e}
 form{display:flex;gap:8px;padding:10px 12px;background:#1b1b1b;border-top:1px solid #333}
 textarea{flex:1;min-height:48px;background:#222;color:#ddd;border:1px solid #444;border-radius:4px;padding:6px}
 button{background:#2d5fa8;color:#fff;border:0;border-radius:4px;padding:0 16px;cursor:pointer}
 button:disabled{background:#444}
 #stat{margin-left:auto;color:#8a8a8a}
</style></head><body>
<header>
 <b>ninfer-fusion-b200</b>
 <label>key <input id="key" type="password" size="14" placeholder="API key"></label>
 <label>max tokens <input id="maxtok" type="number" value="256" min="1" max="8192" style="width:70px"></label>
 <label>temperature <input id="temp" type="number" value="0.7" step="0.1" min="0" max="2" style="width:60px"></label>
 <label><input id="think" type="checkbox"> thinking</label>
 <button id="clear" type="button">new chat</button>
 <span id="stat">connecting</span>
</header>
<div id="log"></div>
<form id="f"><textarea id="in" placeholder="Message (Ctrl+Enter to send)"></textarea><button id="send">Send</button></form>
<script>
const $=id=>document.getElementById(id);let messages=[];let model="";
function hdr(){const h={"Content-Type":"application/json"};if($("key").value)h["Authorization"]="Bearer "+$("key").value;return h}
function add(cls,text){const d=document.createElement("div");d.className="msg "+cls;d.textContent=text;$("log").appendChild(d);$("log").scrollTop=1e9;return d}
async function probe(){try{const h=await (await fetch("/health")).json();let t=h.status||"ok";
 const m=await fetch("/v1/models",{headers:hdr()});if(m.ok){model=(await m.json()).data[0].id;t+=" | "+model}else{t+=" | key needed"}
 $("stat").textContent=t}catch(e){$("stat").textContent="server unreachable"}}
$("key").addEventListener("change",probe);$("clear").onclick=()=>{messages=[];$("log").textContent=""};
$("in").addEventListener("keydown",e=>{if(e.key==="Enter"&&(e.ctrlKey||e.metaKey)){e.preventDefault();$("f").requestSubmit()}});
$("f").addEventListener("submit",async e=>{e.preventDefault();const text=$("in").value.trim();if(!text)return;
 $("in").value="";$("send").disabled=true;messages.push({role:"user",content:text});add("user",text);
 const think=add("assistant think","");think.style.display="none";const out=add("assistant","");let answer="";const t0=performance.now();let n=0;
 try{const r=await fetch("/v1/chat/completions",{method:"POST",headers:hdr(),body:JSON.stringify({model:model,messages:messages,stream:true,
   max_tokens:+$("maxtok").value,temperature:+$("temp").value,enable_thinking:$("think").checked})});
  if(!r.ok){const j=await r.json().catch(()=>({}));throw new Error((j.error&&j.error.message)||("HTTP "+r.status))}
  const rd=r.body.getReader();const dec=new TextDecoder();let buf="";
  for(;;){const {done,value}=await rd.read();if(done)break;buf+=dec.decode(value,{stream:true});let i;
   while((i=buf.indexOf("\\n\\n"))>=0){const block=buf.slice(0,i);buf=buf.slice(i+2);
    for(const line of block.split("\\n")){if(!line.startsWith("data: "))continue;const p=line.slice(6);if(p==="[DONE]")continue;
     const d=JSON.parse(p).choices[0].delta||{};if(d.reasoning_content){think.style.display="";think.textContent+=d.reasoning_content}
     if(d.content){answer+=d.content;out.textContent=answer;n++}$("log").scrollTop=1e9}}}
  messages.push({role:"assistant",content:answer});
  $("stat").textContent=model+" | "+n+" chunks in "+((performance.now()-t0)/1000).toFixed(1)+" s";
 }catch(err){out.className="msg err";out.textContent=String(err.message||err);messages.pop()}
 $("send").disabled=false;$("in").focus()});
probe();
</script></body></html>
"""


def page_bytes() -> bytes:
    return PAGE.encode("utf-8")
