/* A host in plain C11 over the C ABI: what a cgo / JNI / Rust-FFI binding sees.  Compiled and linked by
 * tests/test_abi.py with gcc -std=c11 -pedantic (no C++ anywhere on this side); it calls only entry points that need no
 * device, so it runs on any machine: the version, the scheduler with its eviction planner, the attention planner, the
 * sampler's random numbers. */
#include <stdio.h>
#include <string.h>

#include "eb_synth.h"
#include "eidola_b200.h"

int main(void) {
  int32_t abi = 0;
  if (eb_version(&abi) != EB_OK || abi != EB_ABI_VERSION) return 1;
  eb_sched* s = NULL;
  if (eb_sched_create(64, 16, 4, 8, 0, &s) != EB_OK) return 2;
  int32_t slot = -1;
  if (eb_sched_admit(s, 40, &slot) != EB_OK || slot < 0) return 3;
  if (eb_sched_extend(s, slot, 45) != EB_OK) return 4;
  int32_t slots[1], q_lens[1] = {5}, q_off[2], ctx[1], tok_seq[5], tok_slot[5], pos[5], n_tok = 0;
  slots[0] = slot;
  if (eb_sched_pack(s, slots, q_lens, 1, q_off, ctx, tok_seq, tok_slot, pos, &n_tok) != EB_OK) return 5;
  if (n_tok != 5 || ctx[0] != 45 || pos[0] != 40 || pos[4] != 44) return 6;
  eb_attn_item items[16];
  int32_t n_items = 0, seq_part[2], n_parts = 0;
  const int32_t plan_sms = eb_attn_plan_sm_count(148, 5, 64, 8, 0);
  if (eb_attn_plan(ctx, q_lens, 1, 16, 0, plan_sms, 0, 1, items, 16, &n_items, seq_part, &n_parts) != EB_OK) return 7;
  if (n_items < 1 || items[0].page_begin != 0 || seq_part[1] != n_parts) return 8;
  if (eb_sample_rand32(1, 2) == eb_sample_rand32(1, 3)) return 9;
  char msg[256];
  eb_sched_admit(s, 1 << 30, &slot); /* refused: the message names the reason */
  eb_last_error(msg, sizeof msg);
  if (strlen(msg) == 0) return 10;
  if (eb_sched_destroy(s) != EB_OK) return 11;
  printf("c host ok: abi %d, %d work items, bf16(1.0f) = 0x%04x\n", (int)abi, (int)n_items, (unsigned)eb_bf16_from_f32(1.0f));
  return 0;
}
