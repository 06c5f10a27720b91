"""Minimal chat web UI (reference: ``ftllm webui``, a Streamlit page on port 1616).  Served as a single static page by
the same FastAPI app as the API, so it needs no extra dependency; it talks to ``/v1/chat/completions`` with streaming."""
from __future__ import annotations

PAGE = """<!doctype html><html><head><meta charset="utf-8"><title>fastllm_b200</title>
<style>body{font-family:sans-serif;max-width:760px;margin:2em auto}#log div{margin:.6em 0;white-space:pre-wrap}
.u{color:#024}.a{color:#040}textarea{width:100%;height:5em}</style></head><body><h3>fastllm_b200 chat</h3>
<div id="log"></div><textarea id="q" placeholder="message"></textarea><button onclick="send()">send</button>
<script>
const msgs=[];async function send(){const q=document.getElementById('q');const t=q.value;if(!t)return;q.value='';
msgs.push({role:'user',content:t});add('u','User: '+t);const el=add('a','AI: ');
const r=await fetch('/v1/chat/completions',{method:'POST',headers:{'Content-Type':'application/json'},
body:JSON.stringify({messages:msgs,stream:true})});const rd=r.body.getReader();const dec=new TextDecoder();let buf='',out='';
while(true){const {done,value}=await rd.read();if(done)break;buf+=dec.decode(value,{stream:true});
let i;while((i=buf.indexOf('\\n\\n'))>=0){const line=buf.slice(0,i);buf=buf.slice(i+2);
if(!line.startsWith('data: ')||line.includes('[DONE]'))continue;const d=JSON.parse(line.slice(6)).choices[0].delta;
if(d.content){out+=d.content;el.textContent='AI: '+out;}}}msgs.push({role:'assistant',content:out});}
function add(c,t){const d=document.createElement('div');d.className=c;d.textContent=t;document.getElementById('log').appendChild(d);return d;}
</script></body></html>"""


def run_webui(args):
    import uvicorn
    from fastapi.responses import HTMLResponse

    from ..util import make_normal_llm_model
    from .server import build_app

    model = make_normal_llm_model(args)
    app = build_app(model, args.model_name or "fastllm-b200", args.api_key)

    @app.get("/", response_class=HTMLResponse)
    async def index():
        return PAGE

    uvicorn.run(app, host=args.host, port=args.port if args.port != 8080 else 1616, log_level="warning")
