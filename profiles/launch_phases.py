"""Per-kernel device time of ONE prompt pass and ONE decode step from an ncu launch list of bench.py --compare-families."""
import csv,re,collections,sys
f=sys.argv[1]; T=sys.argv[2]; B=sys.argv[3]
rows=list(csv.reader(open(f)))
hi=next(i for i,r in enumerate(rows) if 'Kernel Name' in r)
hdr=rows[hi]
ki=hdr.index('Kernel Name'); vi=hdr.index('Metric Value'); gi=hdr.index('Grid Size')
# passes are delimited by the embedding kernel
seq=[]
for r in rows[hi+1:]:
    if len(r)<=vi: continue
    n=re.sub(r'\(.*','',r[ki]).replace('void ','')
    if not (n.startswith('hy_') or n.startswith('xb_')): continue
    if 'load_convert' in n or 'tile_weight' in n: continue
    seq.append((n[:52], r[gi], float(r[vi].replace(',',''))/1000))
passes=[]; cur=None
for n,g,t in seq:
    if 'embed' in n:
        cur={'grid':g,'k':collections.OrderedDict()}; passes.append(cur)
    if cur is None: continue
    a=cur['k'].setdefault(n,[0,0.0]); a[0]+=1; a[1]+=t
def show(tag, sel):
    ps=[p for p in passes if sel(p)]
    if not ps: return
    p=ps[-1]
    tot=sum(a[1] for a in p['k'].values()); nl=sum(a[0] for a in p['k'].values())
    print(f"== {tag}: {nl} launches, {tot:.0f} us (ncu, cold caches, serialised)")
    for n,(c,t) in sorted(p['k'].items(), key=lambda kv:-kv[1][1]):
        print(f"  {t:8.1f} us {100*t/tot:5.1f}%  n={c:3d} avg={t/c:7.1f}  {n}")
show(f"prompt of {T} tokens", lambda p: p['grid'].startswith(f'({T},'))
show(f"decode step, {B} sequences", lambda p: p['grid'].startswith(f'({B},'))
