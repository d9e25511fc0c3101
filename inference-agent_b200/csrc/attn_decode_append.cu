// K1 + K3 for one token in one launch: the decode kernel of attn_decode.cu compiled in its "append" form (RoPE on q and
// on the new k, K/V row appended by the CTA that owns it, attention over all keys including the new one).
// See the note at the top of attn_decode.cu.
#define INGOT_DECODE_APPEND 1
#include "attn_decode.cu"
