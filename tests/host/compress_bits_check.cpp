// Host build of the pure bit helpers of the compression kernels (mustafar_b200/csrc/compress_bits.cuh):
// the 16x16 bit transposes, the plane-to-bitmap reordering, the byte interleave of a thread pair, the
// warp-wide 32x32 transpose (emulated over 32 "lanes") and the bit-sliced radix select, each against
// a plain loop.  Built and run by tests/test_host_bits.py with g++; prints "ok" and exits 0.
#include <algorithm>
#include <vector>
#include <cstdio>
#include <cstdlib>
#include <cstdint>
static inline unsigned __byte_perm(unsigned x, unsigned y, unsigned s){
  uint64_t v = ((uint64_t)y<<32)|x; unsigned r=0;
  for(int i=0;i<4;i++){ unsigned sel=(s>>(4*i))&7; r |= (unsigned)((v>>(8*sel))&0xff) << (8*i);} return r; }
static inline unsigned __brev(unsigned x){unsigned r=0;for(int i=0;i<32;i++) if(x>>i&1) r|=1u<<(31-i);return r;}
static inline int __popc(unsigned x){return __builtin_popcount(x);}
#define MFAR_BITS_FN static inline
#include "compress_bits.cuh"
using namespace mfar;
int main(){
  srand(3);
  for(int it=0;it<20000;it++){
    unsigned short row[128]; for(int i=0;i<128;i++) row[i]= (rand()%10<3)? (rand()&0x7fff)|1 : 0;
    // per thread planes -> nonzero flags in plane layout
    unsigned Y[2][2];
    for(int hh=0;hh<2;hh++)for(int g=0;g<2;g++){
      unsigned a[16];
      for(int k=0;k<4;k++){ int chunk=8*g+2*k+hh; for(int j=0;j<4;j++){ int e=chunk*8+2*j; a[4*k+j]=row[e]|((unsigned)row[e+1]<<16);} }
      transpose16x16x2(a);
      unsigned X=0; for(int b=0;b<15;b++) X|=a[b];
      Y[hh][g]=plane_to_bitmap_order(X);
    }
    for(int g=0;g<2;g++){
      unsigned hi,lo; interleave_chunk_bytes(Y[0][g],Y[1][g],hi,lo);
      uint64_t bm=((uint64_t)hi<<32)|lo, ref=0;
      for(int i=0;i<64;i++) if(row[64*g+i]) ref|=1ull<<(63-i);
      if(bm!=ref){printf("mismatch g=%d %016llx %016llx\n",g,(unsigned long long)bm,(unsigned long long)ref);return 1;}
    }
  }
  // warp 32x32 transpose emulation
  for(int it=0;it<1000;it++){
    unsigned x[32],o[32]; for(int i=0;i<32;i++){x[i]=((unsigned)rand()<<16)^rand(); o[i]=x[i];}
    for(int s=16;s>=1;s>>=1){ unsigned m = s==16?0x0000ffffu: s==8?0x00ff00ffu: s==4?0x0f0f0f0fu: s==2?0x33333333u:0x55555555u;
      unsigned n[32]; for(int l=0;l<32;l++){ unsigned y=x[l^s]; n[l]= (l&s)? (((y>>s)&m)|(x[l]&~m)) : ((x[l]&m)|((y<<s)&~m)); }
      for(int l=0;l<32;l++)x[l]=n[l]; }
    for(int i=0;i<32;i++)for(int j=0;j<32;j++) if(((o[i]>>j)&1)!=((x[j]>>i)&1)){printf("warp transpose mismatch\n");return 1;}
  }
  // bit-sliced radix select over a thread pair (2 x 64 values) against a sort
  for(int it=0;it<50000;it++){
    unsigned short v[128]; int mode=it%4;
    for(int i=0;i<128;i++){ v[i]= mode==0? rand()&0x7fff : mode==1? (rand()&0x3f)|0x3c00 : mode==2 ? (rand()%3)*0x1000 : (rand()&0x7fff)>>(rand()%15); }
    int rank=1+rand()%128;
    unsigned pl[2][2][16];
    for(int t=0;t<2;t++)for(int ch=0;ch<2;ch++){ for(int j=0;j<16;j++){int e=t*64+ch*32+2*j; pl[t][ch][j]=v[e]|((unsigned)v[e+1]<<16);} transpose16x16x2(pl[t][ch]); }
    unsigned c[2][2]={{~0u,~0u},{~0u,~0u}}, g[2][2]={{0,0},{0,0}}; int r=rank; unsigned T=0;
    for(int b=14;b>=0;b--){
      int cnt=0; unsigned z[2][2];
      for(int t=0;t<2;t++)for(int ch=0;ch<2;ch++){ z[t][ch]=c[t][ch]&~pl[t][ch][b]; cnt+=__popc(z[t][ch]); }
      const bool zero_side = r<=cnt;
      for(int t=0;t<2;t++)for(int ch=0;ch<2;ch++){ unsigned o=c[t][ch]^z[t][ch]; if(zero_side){g[t][ch]|=o;c[t][ch]=z[t][ch];} else c[t][ch]=o; }
      if(!zero_side){ r-=cnt; T|=1u<<b; }
    }
    std::vector<unsigned short> s(v,v+128); std::sort(s.begin(),s.end());
    if(s[rank-1]!=T){printf("select mismatch\n");return 1;}
    // keep flags: element kept iff value >= T; plane layout bit j = low half of register j, 16+j = high half
    for(int t=0;t<2;t++)for(int ch=0;ch<2;ch++){ unsigned keep=g[t][ch]|c[t][ch];
      for(int j=0;j<16;j++)for(int hf=0;hf<2;hf++){ int e=t*64+ch*32+2*j+hf; bool k=(keep>>(j+16*hf))&1; if(k!=(v[e]>=T)){printf("keep mismatch\n");return 1;} } }
  }
  printf("ok\n");
}
