// The C ABI of libkb200.so: descriptor validation, buffer binding with bounds checks, launch
// dispatch.  Declared and documented in include/kb200.h.
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <new>

#include "kb200_internal.h"

#define KB200_EXPORT extern "C" __attribute__((visibility("default")))

namespace kb200 {

static thread_local std::string g_error;

int fail(int status, const char* fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof buf, fmt, ap);
  va_end(ap);
  g_error = buf;
  return status;
}

int cuda_fail(cudaError_t e, const char* what) {
  return fail(KB200_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
}

const char* impl_name(int impl) {
  static const char* names[IMPL_COUNT] = {
      "ew_generic", "ew_chain_vec4", "ew_transpose", "row_generic", "row_layernorm", "row_softmax",
      "reduce_generic", "mm_simt_fp32", "mm_gemv", "mm_tcgen05", "attention_fused", "fused_away"};
  return impl >= 0 && impl < IMPL_COUNT ? names[impl] : "?";
}

// ---------------------------------------------------------------------------------------------
// Tape analysis
// ---------------------------------------------------------------------------------------------

static bool is_binary(int op) { return op >= KB200_OP_ADD && op <= KB200_OP_MIN; }
static bool is_unary(int op) { return op >= KB200_OP_NEG && op <= KB200_OP_COPY; }
static bool is_reduce(int op) { return op == KB200_OP_RSUM || op == KB200_OP_RMAX; }

static void use_counts(const kb200_kernel_desc& d, int* uses) {
  for (int i = 0; i < d.n_tape; ++i) uses[i] = 0;
  for (int i = 0; i < d.n_tape; ++i) {
    const kb200_tape_op& t = d.tape[i];
    if (is_binary(t.opcode)) { uses[t.a]++; uses[t.b]++; }
    else if (is_unary(t.opcode) || is_reduce(t.opcode) || t.opcode == KB200_OP_STORE) uses[t.a]++;
  }
}

static int chain_unary(int op) {
  switch (op) {
    case KB200_OP_NEG: return CH_NEG;
    case KB200_OP_RELU: return CH_RELU;
    case KB200_OP_EXP: return CH_EXP;
    case KB200_OP_TANH: return CH_TANH;
    case KB200_OP_SIGMOID: return CH_SIGMOID;
    case KB200_OP_ERF: return CH_ERF;
    case KB200_OP_GELU_TANH: return CH_GELU_TANH;
    case KB200_OP_GELU_ERF: return CH_GELU_ERF;
    case KB200_OP_RSQRT: return CH_RSQRT;
    case KB200_OP_SQRT: return CH_SQRT;
    default: return CH_COPY;
  }
}

static int chain_binary(int op, bool reversed) {
  switch (op) {
    case KB200_OP_ADD: return CH_ADD;
    case KB200_OP_SUB: return reversed ? CH_RSUB : CH_SUB;
    case KB200_OP_MUL: return CH_MUL;
    case KB200_OP_DIV: return reversed ? CH_RDIV : CH_DIV;
    case KB200_OP_MAX: return CH_MAX;
    default: return CH_MIN;
  }
}

// A tape is a chain when it has one STORE and every computed value feeds exactly the next op.
bool extract_chain(const kb200_kernel_desc& d, Chain* out) {
  int uses[KB200_MAX_TAPE];
  use_counts(d, uses);
  int store = -1, n_ops = 0;
  for (int i = 0; i < d.n_tape; ++i) {
    int op = d.tape[i].opcode;
    if (op == KB200_OP_STORE) {
      if (store >= 0) return false;
      store = i;
    } else if (is_reduce(op)) {
      return false;
    } else if (is_binary(op) || is_unary(op)) {
      ++n_ops;
    }
  }
  if (store < 0 || n_ops > kMaxChain) return false;
  ChainStep rev[kMaxChain];
  int n = 0;
  int cur = d.tape[store].a;
  auto leaf_side = [&](int i) { int o = d.tape[i].opcode; return o == KB200_OP_LOAD || o == KB200_OP_IMM; };
  auto leaf = [&](int i) { return leaf_side(i) || d.tape[i].opcode == KB200_OP_ACC; };
  auto side_of = [&](int i, ChainStep* s) {
    if (d.tape[i].opcode == KB200_OP_IMM) { s->slot = -1; s->imm = d.tape[i].imm; }
    else { s->slot = d.tape[i].a; s->imm = 0.f; }
  };
  while (true) {
    const kb200_tape_op& e = d.tape[cur];
    if (e.opcode == KB200_OP_LOAD) { out->first_slot = e.a; break; }
    if (e.opcode == KB200_OP_ACC) { out->first_slot = -1; break; }
    if (e.opcode == KB200_OP_IMM) return false;
    if (uses[cur] != 1) return false;
    ChainStep s{};
    int next;
    if (is_unary(e.opcode)) {
      s.op = chain_unary(e.opcode);
      s.slot = -2;
      next = e.a;
    } else {
      bool a_leaf = leaf(e.a), b_leaf = leaf(e.b);
      int main_i, side_i;
      bool reversed;
      if (a_leaf && b_leaf) {
        bool a_acc = d.tape[e.a].opcode == KB200_OP_ACC, b_acc = d.tape[e.b].opcode == KB200_OP_ACC;
        if (a_acc && b_acc) return false;
        if (b_acc || (!a_acc && d.tape[e.a].opcode == KB200_OP_IMM)) { main_i = e.b; side_i = e.a; reversed = true; }
        else { main_i = e.a; side_i = e.b; reversed = false; }
        if (d.tape[main_i].opcode == KB200_OP_IMM) return false;
      } else if (b_leaf && leaf_side(e.b)) { main_i = e.a; side_i = e.b; reversed = false; }
      else if (a_leaf && leaf_side(e.a)) { main_i = e.b; side_i = e.a; reversed = true; }
      else return false;
      if (main_i == side_i) return false;
      s.op = chain_binary(e.opcode, reversed);
      side_of(side_i, &s);
      next = main_i;
    }
    if (n >= kMaxChain) return false;
    rev[n++] = s;
    cur = next;
  }
  if (n != n_ops) return false;   // some op is off the chain
  out->n = n;
  out->out_slot = d.tape[store].b;
  for (int i = 0; i < n; ++i) out->steps[i] = rev[n - 1 - i];
  return true;
}

namespace {
struct Matcher {
  const kb200_kernel_desc& d;
  const kb200_tape_op& at(int i) const { return d.tape[i]; }
  bool is(int i, int op) const { return d.tape[i].opcode == op; }
  // For a commutative binary op at i: find the argument satisfying pred, return it and the other one.
  template <class P>
  bool split(int i, int op, P pred, int* hit, int* other) const {
    if (!is(i, op)) return false;
    if (pred(at(i).a)) { *hit = at(i).a; *other = at(i).b; return true; }
    if (pred(at(i).b)) { *hit = at(i).b; *other = at(i).a; return true; }
    return false;
  }
};
}  // namespace

// The value `z` a row kernel reduces over: a LOAD, or a short chain of elementwise ops on one (every
// step a unary op, or a binary op whose other argument is a LOAD or an immediate), as in
// softmax(x * scale + mask) or LayerNorm(a + b).  Fills first slot and steps; *entries counts the
// tape entries the chain consists of (the first LOAD, the ops, their leaves).
static bool row_pre_chain(const kb200_kernel_desc& d, int z, Chain* out, int* entries) {
  ChainStep rev[kMaxRowPre];
  int n = 0, count = 0, cur = z;
  auto leaf = [&](int i) { return d.tape[i].opcode == KB200_OP_LOAD || d.tape[i].opcode == KB200_OP_IMM; };
  while (d.tape[cur].opcode != KB200_OP_LOAD) {
    const kb200_tape_op& e = d.tape[cur];
    if (n >= kMaxRowPre) return false;
    ChainStep s{};
    if (is_unary(e.opcode)) {
      s.op = chain_unary(e.opcode);
      s.slot = -2;
      cur = e.a;
    } else if (is_binary(e.opcode)) {
      int main_i, side_i;
      bool reversed;
      if (leaf(e.b) && d.tape[e.a].opcode != KB200_OP_IMM) { main_i = e.a; side_i = e.b; reversed = false; }
      else if (leaf(e.a) && d.tape[e.b].opcode != KB200_OP_IMM) { main_i = e.b; side_i = e.a; reversed = true; }
      else return false;
      s.op = chain_binary(e.opcode, reversed);
      if (d.tape[side_i].opcode == KB200_OP_IMM) { s.slot = -1; s.imm = d.tape[side_i].imm; }
      else { s.slot = d.tape[side_i].a; }
      ++count;                      // the leaf
      cur = main_i;
    } else {
      return false;
    }
    ++count;                        // the op
    rev[n++] = s;
  }
  out->first_slot = d.tape[cur].a;
  out->n = n;
  for (int i = 0; i < n; ++i) out->steps[i] = rev[n - 1 - i];
  *entries = count + 1;             // + the first LOAD
  return true;
}

// y = (x - mean) * rsqrt(var + eps) * gamma + beta with the two-pass mean / variance the frontend
// emits (kiln/frontend/fx_import.py:217-230); x a loaded row or a short chain on one (a residual add
// fused in front), which may itself be stored as a second output.
bool match_layernorm(const kb200_kernel_desc& d, PlanKernel* k) {
  Matcher m{d};
  int stores = 0, st = -1, reduces = 0;
  for (int i = 0; i < d.n_tape; ++i) {
    if (m.is(i, KB200_OP_STORE)) ++stores;
    if (is_reduce(d.tape[i].opcode)) ++reduces;
  }
  if (stores < 1 || stores > 2 || reduces != 2) return false;
  // the LayerNorm's own store is the one at the deepest level (after both reductions)
  for (int i = 0; i < d.n_tape; ++i)
    if (m.is(i, KB200_OP_STORE) && (st < 0 || d.tape[i].level > d.tape[st].level)) st = i;
  auto is_load = [&](int i) { return m.is(i, KB200_OP_LOAD); };
  auto is_imm = [&](int i) { return m.is(i, KB200_OP_IMM); };
  int beta, y1, gamma, y0;
  if (!m.split(m.at(st).a, KB200_OP_ADD, is_load, &beta, &y1)) return false;
  if (!m.split(y1, KB200_OP_MUL, is_load, &gamma, &y0)) return false;
  if (!m.is(y0, KB200_OP_MUL)) return false;
  int xc = m.at(y0).a, rstd = m.at(y0).b;
  if (!m.is(xc, KB200_OP_SUB)) { int t = xc; xc = rstd; rstd = t; }
  if (!m.is(xc, KB200_OP_SUB) || !m.is(rstd, KB200_OP_RSQRT)) return false;
  int x = m.at(xc).a, mean = m.at(xc).b;
  Chain pre{};
  int pre_entries = 0;
  if (!row_pre_chain(d, x, &pre, &pre_entries)) return false;
  int pre_out = -1;
  for (int i = 0; i < d.n_tape; ++i)
    if (m.is(i, KB200_OP_STORE) && i != st) {
      if (m.at(i).a != x || pre.n == 0) return false;      // the second output must be the chain's value
      pre_out = m.at(i).b;
    }
  // nothing else in the tape: 16 entries of the LayerNorm proper beside x, the chain, the stores
  if (d.n_tape != 16 + pre_entries + (stores - 1)) return false;
  int c1, s1;
  if (!m.split(mean, KB200_OP_MUL, is_imm, &c1, &s1)) return false;
  if (!m.is(s1, KB200_OP_RSUM) || m.at(s1).a != x) return false;
  int eps, var;
  if (!m.split(m.at(rstd).a, KB200_OP_ADD, is_imm, &eps, &var)) return false;
  int c2, s2;
  if (!m.split(var, KB200_OP_MUL, is_imm, &c2, &s2)) return false;
  if (!m.is(s2, KB200_OP_RSUM)) return false;
  int sq = m.at(s2).a;
  if (!m.is(sq, KB200_OP_MUL) || m.at(sq).a != xc || m.at(sq).b != xc) return false;
  if (m.at(c1).imm != m.at(c2).imm) return false;
  k->x_slot = pre.first_slot;
  k->row_pre = pre;
  k->pre_out_slot = pre_out;
  k->g_slot = m.at(gamma).a;
  k->b_slot = m.at(beta).a;
  k->out_slot = m.at(st).b;
  k->ln_inv_n = m.at(c1).imm;
  k->ln_eps = m.at(eps).imm;
  return true;
}

// out = exp(x - max(x)) / sum(exp(x - max(x))) (kiln/frontend/fx_import.py:212-216).
bool match_softmax(const kb200_kernel_desc& d, PlanKernel* k) {
  Matcher m{d};
  int st = d.n_tape - 1, stores = 0;
  for (int i = 0; i < d.n_tape; ++i)
    if (m.is(i, KB200_OP_STORE)) ++stores;
  if (stores != 1 || !m.is(st, KB200_OP_STORE)) return false;
  int dv = m.at(st).a;
  if (!m.is(dv, KB200_OP_DIV)) return false;
  int e = m.at(dv).a, s = m.at(dv).b;
  if (!m.is(e, KB200_OP_EXP) || !m.is(s, KB200_OP_RSUM) || m.at(s).a != e) return false;
  int sub = m.at(e).a;
  if (!m.is(sub, KB200_OP_SUB)) return false;
  int x = m.at(sub).a, mx = m.at(sub).b;
  if (!m.is(mx, KB200_OP_RMAX) || m.at(mx).a != x) return false;
  // x: the loaded row, or a short chain on it (scale and additive mask fused in front)
  Chain pre{};
  int pre_entries = 0;
  if (!row_pre_chain(d, x, &pre, &pre_entries)) return false;
  if (d.n_tape != 6 + pre_entries) return false;
  k->x_slot = pre.first_slot;
  k->row_pre = pre;
  k->pre_out_slot = -1;
  k->out_slot = m.at(st).b;
  return true;
}

// ---------------------------------------------------------------------------------------------
// Validation
// ---------------------------------------------------------------------------------------------

static int validate(const kb200_kernel_desc& d, int index) {
  const char* nm = d.name;
  if (d.kclass < KB200_K_ELEMENTWISE || d.kclass > KB200_K_MATMUL)
    return fail(KB200_ERR_ARGUMENT, "kernel %d (%s): unknown class %d", index, nm, d.kclass);
  if (d.iter_rank < 1 || d.iter_rank > KB200_MAX_RANK)
    return fail(KB200_ERR_ARGUMENT, "kernel %d (%s): iteration rank %d out of range", index, nm, d.iter_rank);
  if (d.n_operands < 1 || d.n_operands > KB200_MAX_OPERANDS)
    return fail(KB200_ERR_ARGUMENT, "kernel %d (%s): %d operands out of range", index, nm, d.n_operands);
  if (d.n_tape < 1 || d.n_tape > KB200_MAX_TAPE)
    return fail(KB200_ERR_ARGUMENT, "kernel %d (%s): tape length %d out of range", index, nm, d.n_tape);
  if (d.precision < KB200_PREC_FP32 || d.precision > KB200_PREC_BF16)
    return fail(KB200_ERR_ARGUMENT, "kernel %d (%s): unknown precision %d", index, nm, d.precision);
  for (int i = 0; i < d.iter_rank; ++i)
    if (d.iter_shape[i] < 0 || d.iter_shape[i] > (int64_t(1) << 40))
      return fail(KB200_ERR_ARGUMENT, "kernel %d (%s): bad extent %lld", index, nm, (long long)d.iter_shape[i]);
  for (int o = 0; o < d.n_operands; ++o) {
    const kb200_operand& op = d.operands[o];
    if (op.base_kind < KB200_BASE_ARENA || op.base_kind > KB200_BASE_OUTPUT || op.base_index < 0 || op.elem_offset < 0)
      return fail(KB200_ERR_ARGUMENT, "kernel %d (%s): operand %d has a bad base or offset", index, nm, o);
    for (int i = 0; i < KB200_MAX_RANK; ++i)
      if (op.stride[i] < 0)
        return fail(KB200_ERR_UNSUPPORTED, "kernel %d (%s): operand %d has a negative stride", index, nm, o);
  }
  int stores = 0;
  for (int i = 0; i < d.n_tape; ++i) {
    const kb200_tape_op& t = d.tape[i];
    bool ok = true;
    switch (t.opcode) {
      case KB200_OP_LOAD: ok = t.a >= 0 && t.a < d.n_operands; break;
      case KB200_OP_IMM: break;
      case KB200_OP_ACC: ok = d.kclass == KB200_K_MATMUL; break;
      case KB200_OP_STORE:
        ok = t.a >= 0 && t.a < i && t.b >= 0 && t.b < d.n_operands && d.tape[t.a].opcode != KB200_OP_STORE;
        ++stores;
        break;
      case KB200_OP_RSUM:
      case KB200_OP_RMAX:
        ok = (d.kclass == KB200_K_ROW || d.kclass == KB200_K_REDUCE) && t.a >= 0 && t.a < i;
        break;
      default:
        if (is_binary(t.opcode)) ok = t.a >= 0 && t.a < i && t.b >= 0 && t.b < i;
        else if (is_unary(t.opcode)) ok = t.a >= 0 && t.a < i;
        else return fail(KB200_ERR_UNSUPPORTED, "kernel %d (%s): no lowering for opcode %d", index, nm, t.opcode);
    }
    if (!ok) return fail(KB200_ERR_ARGUMENT, "kernel %d (%s): tape entry %d is malformed", index, nm, i);
    if ((is_binary(t.opcode) && (d.tape[t.a].opcode == KB200_OP_STORE || d.tape[t.b].opcode == KB200_OP_STORE)) ||
        ((is_unary(t.opcode) || is_reduce(t.opcode)) && d.tape[t.a].opcode == KB200_OP_STORE))
      return fail(KB200_ERR_ARGUMENT, "kernel %d (%s): tape entry %d reads a STORE", index, nm, i);
    if (t.level < 0 || t.level > 16)
      return fail(KB200_ERR_ARGUMENT, "kernel %d (%s): tape entry %d has level %d", index, nm, i, t.level);
  }
  if (stores == 0) return fail(KB200_ERR_ARGUMENT, "kernel %d (%s): tape stores nothing", index, nm);
  if (d.kclass == KB200_K_MATMUL) {
    if (d.iter_rank != 3 || d.a_slot < 0 || d.a_slot >= d.n_operands || d.b_slot < 0 || d.b_slot >= d.n_operands ||
        d.a_slot == d.b_slot || d.k_extent < 0)
      return fail(KB200_ERR_ARGUMENT, "kernel %d (%s): malformed matmul descriptor", index, nm);
    if (d.iter_shape[0] > 65535)
      return fail(KB200_ERR_UNSUPPORTED, "kernel %d (%s): matmul batch %lld exceeds CUDA grid limits", index, nm,
                  (long long)d.iter_shape[0]);
  }
  if (d.kclass == KB200_K_REDUCE) {
    if (d.n_kept < 0 || d.n_kept > d.iter_rank || d.n_tape != 3 || d.tape[0].opcode != KB200_OP_LOAD ||
        !is_reduce(d.tape[1].opcode) || d.tape[2].opcode != KB200_OP_STORE)
      return fail(KB200_ERR_ARGUMENT, "kernel %d (%s): malformed reduction descriptor", index, nm);
  }
  return KB200_OK;
}

// Checks that every element an operand can reach lies inside the buffer it is bound to.
static int check_span(const Plan& plan, const kb200_kernel_desc& d, int index, int slot, const int64_t* extents,
                      int rank, uint64_t bytes) {
  const kb200_operand& op = d.operands[slot];
  int64_t last = op.elem_offset;
  for (int i = 0; i < rank; ++i) {
    if (extents[i] == 0) return KB200_OK;  // nothing is touched
    last += (extents[i] - 1) * op.stride[i];
  }
  if (uint64_t(last + 1) * 4 > bytes)
    return fail(KB200_ERR_BOUNDS, "kernel %d (%s): operand %d reaches element %lld but its buffer holds %llu bytes", index,
                d.name, slot, (long long)last, (unsigned long long)bytes);
  (void)plan;
  return KB200_OK;
}

static int resolve(Plan& plan, PlanKernel& k, int index) {
  const kb200_kernel_desc& d = k.desc;
  for (int o = 0; o < d.n_operands; ++o) {
    const kb200_operand& op = d.operands[o];
    float* base = nullptr;
    uint64_t bytes = 0;
    auto pick = [&](const std::vector<float*>& ptrs, const std::vector<uint64_t>& sizes, const char* what) -> int {
      if (op.base_index >= (int)ptrs.size())
        return fail(KB200_ERR_ARGUMENT, "kernel %d (%s): operand %d names %s %d but only %d were bound", index, d.name, o,
                    what, op.base_index, (int)ptrs.size());
      base = ptrs[op.base_index];
      bytes = sizes[op.base_index];
      return KB200_OK;
    };
    int rc = KB200_OK;
    switch (op.base_kind) {
      case KB200_BASE_ARENA: base = plan.arena; bytes = plan.arena_bytes; break;
      case KB200_BASE_CONST: rc = pick(plan.consts, plan.const_bytes, "constant"); break;
      case KB200_BASE_INPUT: rc = pick(plan.inputs, plan.input_bytes, "input"); break;
      default: rc = pick(plan.outputs, plan.output_bytes, "output"); break;
    }
    if (rc) return rc;
    if (base == nullptr) return fail(KB200_ERR_ARGUMENT, "kernel %d (%s): operand %d is bound to a null buffer", index, d.name, o);
    int64_t ext[KB200_MAX_RANK];
    int rank = d.iter_rank;
    for (int i = 0; i < rank; ++i) ext[i] = d.iter_shape[i];
    if (d.kclass == KB200_K_MATMUL) {
      if (o == d.a_slot) { ext[2] = d.k_extent; }
      else if (o == d.b_slot) { ext[1] = d.k_extent; ext[2] = d.iter_shape[2]; }
    }
    rc = check_span(plan, d, index, o, ext, rank, bytes);
    if (rc) return rc;
    k.ops[o].ptr = base + op.elem_offset;
    for (int i = 0; i < KB200_MAX_RANK; ++i) k.ops[o].stride[i] = op.stride[i];
  }
  return KB200_OK;
}

namespace {
struct Span {
  const float* lo;
  const float* hi;
};
Span span_of(const PlanKernel& k, int slot) {
  const kb200_kernel_desc& d = k.desc;
  int64_t ext[KB200_MAX_RANK];
  for (int i = 0; i < d.iter_rank; ++i) ext[i] = d.iter_shape[i];
  if (d.kclass == KB200_K_MATMUL) {
    if (slot == d.a_slot) ext[2] = d.k_extent;
    if (slot == d.b_slot) { ext[1] = d.k_extent; ext[2] = d.iter_shape[2]; }
  }
  int64_t last = 0;
  for (int i = 0; i < d.iter_rank; ++i) last += (ext[i] - 1) * k.ops[slot].stride[i];
  return {k.ops[slot].ptr, k.ops[slot].ptr + last + 1};
}
}  // namespace

namespace {
void reads_and_writes(const PlanKernel& k, std::vector<int>* reads, std::vector<int>* writes) {
  const kb200_kernel_desc& d = k.desc;
  if (d.kclass == KB200_K_MATMUL) {
    reads->push_back(d.a_slot);
    reads->push_back(d.b_slot);
  }
  for (int t = 0; t < d.n_tape; ++t) {
    if (d.tape[t].opcode == KB200_OP_LOAD) reads->push_back(d.tape[t].a);
    if (d.tape[t].opcode == KB200_OP_STORE) writes->push_back(d.tape[t].b);
  }
  for (int slot = d.n_operands; slot < k.n_ops; ++slot) reads->push_back(slot);   // side operands of an absorbed kernel
}
bool spans_overlap(const Span& a, const Span& b) { return a.lo < b.hi && b.lo < a.hi; }
}  // namespace

// The buffer-assignment pass of the reference makes every matmul's B operand N-contiguous, with a
// copy kernel where the value is not (kiln/passes/buffers.py:208-217): unfrozen weights, `x @ y.T`
// on an intermediate, the K^T of attention.  The matmuls here also read a K-contiguous B (the
// tensor-core kernel as a K-major operand, the SIMT kernel through its strides), so when such a copy
// feeds exactly one matmul and nothing else, the matmul reads the copy's SOURCE and the copy is not
// launched.  The plan itself (kernel list, offsets) is untouched.
static void fold_operand_copies(Plan& plan) {
  // A kernel the fused attention covers still stands for reads and writes the fused kernel makes
  // (Q, K, V; the merged output): only copies this pass folded itself may be ignored by the scans below.
  auto covered_by_attention = [&](size_t i) {
    for (size_t back = 1; back <= 6 && back <= i; ++back)
      if (plan.kernels[i - back].impl == IMPL_ATTN_FUSED) return (int)back < attention_chain_length(plan.kernels[i - back]);
    return false;
  };
  for (size_t j = 0; j < plan.kernels.size(); ++j) {
    PlanKernel& m = plan.kernels[j];
    if (m.desc.kclass != KB200_K_MATMUL || m.impl == IMPL_FUSED_AWAY) continue;
    const int bs = m.desc.b_slot;
    if (m.desc.operands[bs].base_kind != KB200_BASE_ARENA) continue;
    const DevOperand B = m.ops[bs];
    const Span b_span = span_of(m, bs);
    // B as the matmul sees it: dense [batch, K, N]
    if (B.stride[2] != 1 || B.stride[1] != m.N || (m.batch > 1 && B.stride[0] != m.K * m.N)) continue;
    // the kernel that wrote it: the nearest earlier one whose output touches it
    size_t ci = plan.kernels.size();
    for (size_t i = j; i-- > 0 && ci == plan.kernels.size();) {
      const PlanKernel& c = plan.kernels[i];
      if (c.impl == IMPL_FUSED_AWAY) continue;
      if (c.impl == IMPL_ATTN_FUSED) break;
      std::vector<int> reads, writes;
      reads_and_writes(c, &reads, &writes);
      for (int slot : writes)
        if (spans_overlap(span_of(c, slot), b_span)) ci = i;
      if (ci == i) break;
    }
    if (ci == plan.kernels.size()) continue;
    PlanKernel& c = plan.kernels[ci];
    const kb200_kernel_desc& cd = c.desc;
    if (cd.kclass != KB200_K_ELEMENTWISE || !c.has_chain || c.chain.n != 1 || c.chain.steps[0].op != CH_COPY || c.chain.first_slot < 0)
      continue;
    {
      std::vector<int> reads, writes;
      reads_and_writes(c, &reads, &writes);
      if (writes.size() != 1) continue;
    }
    const DevOperand& out = c.ops[c.chain.out_slot];
    const DevOperand& src = c.ops[c.chain.first_slot];
    if (out.ptr != B.ptr || numel_of(cd) != m.batch * m.K * m.N) continue;
    // the copy's output must be dense row-major over its iteration space
    int64_t dense = 1;
    bool ok = true;
    for (int d = cd.iter_rank - 1; d >= 0; --d) {
      if (cd.iter_shape[d] > 1 && out.stride[d] != dense) ok = false;
      dense *= cd.iter_shape[d];
    }
    if (!ok) continue;
    // offset in the source of the element that lands `delta` elements into the output
    auto src_offset = [&](int64_t delta) {
      int64_t off = 0;
      for (int d = cd.iter_rank - 1; d >= 0; --d) {
        off += (delta % cd.iter_shape[d]) * src.stride[d];
        delta /= cd.iter_shape[d];
      }
      return off;
    };
    const int64_t s_n = m.N > 1 ? src_offset(1) : 0, s_k = m.K > 1 ? src_offset(m.N) : 0,
                  s_b = m.batch > 1 ? src_offset(m.K * m.N) : 0;
    // ... which must be linear in (batch, k, n): checked on the corners and their neighbours
    for (int64_t bb : {int64_t(0), m.batch - 1})
      for (int64_t kk : {int64_t(0), m.K > 1 ? int64_t(1) : int64_t(0), m.K - 1})
        for (int64_t nn : {int64_t(0), m.N > 1 ? int64_t(1) : int64_t(0), m.N - 1})
          ok = ok && src_offset(bb * m.K * m.N + kk * m.N + nn) == bb * s_b + kk * s_k + nn * s_n;
    if (!ok || s_n < 0 || s_k < 0 || s_b < 0) continue;
    // nothing between the copy and the matmul may rewrite the source, and nobody but this matmul may
    // read the copy before it is rewritten
    const Span src_span = span_of(c, c.chain.first_slot);
    for (size_t i = ci + 1; i < j && ok; ++i) {
      if (plan.kernels[i].impl == IMPL_FUSED_AWAY && !covered_by_attention(i)) continue;
      std::vector<int> reads, writes;
      reads_and_writes(plan.kernels[i], &reads, &writes);
      for (int slot : writes) ok = ok && !spans_overlap(span_of(plan.kernels[i], slot), src_span);
    }
    bool rewritten = false;
    for (size_t i = ci + 1; i < plan.kernels.size() && ok && !rewritten; ++i) {
      const PlanKernel& k = plan.kernels[i];
      if (k.impl == IMPL_FUSED_AWAY && !covered_by_attention(i)) continue;
      std::vector<int> reads, writes;
      reads_and_writes(k, &reads, &writes);
      for (int slot : reads)
        if (!(i == j && slot == bs) && spans_overlap(span_of(k, slot), b_span)) ok = false;
      for (int slot : writes) {
        const Span w = span_of(k, slot);
        if (w.lo <= b_span.lo && w.hi >= b_span.hi) rewritten = true;
        else if (spans_overlap(w, b_span) && i != j) ok = false;
      }
    }
    if (!ok) continue;
    const PlanKernel saved = m;
    m.ops[bs].ptr = src.ptr;
    m.ops[bs].stride[0] = s_b;
    m.ops[bs].stride[1] = s_k;
    m.ops[bs].stride[2] = s_n;
    if (choose_matmul(plan, m) != KB200_OK) {      // (only a forced implementation can refuse the new strides)
      m = saved;
      continue;
    }
    c.impl = IMPL_FUSED_AWAY;
    c.launches = 0;
  }
}


// An elementwise kernel that directly follows a tensor-core matmul and only continues it becomes the
// tail of the matmul's epilogue chain.  The conditions: the matmul's accumulator chain and the
// elementwise kernel's chain fit one chain; exactly one input of the elementwise kernel is the
// matmul's whole output, element for element; its other inputs and its output are linear in the
// matmul's (row, column); nothing else reads the matmul's output before it is rewritten; and the
// output does not lie over anything the matmul still reads (variants (a) and (b) below).  The plan
// (kernel list, offsets) is untouched: the elementwise kernel stays in it and launches nothing.
// The same for the short chain in front of a register-resident row kernel (LayerNorm(x + matmul),
// the residual add before the second LayerNorm of a block): the matmul then writes the chain's value
// -- into the row kernel's second output where it has one, else into its own buffer -- and the row
// kernel reads it from there and keeps its reductions only.
static void absorb_elementwise(Plan& plan) {
  // from the last matmul to the first: what a later matmul no longer writes (its own output, once it
  // has taken over an elementwise kernel's) is known when an earlier one looks at its readers
  for (size_t j = plan.kernels.size() > 1 ? plan.kernels.size() - 1 : 0; j-- > 0;) {
    PlanKernel& m = plan.kernels[j];
    PlanKernel& e = plan.kernels[j + 1];
    if (m.impl != IMPL_MM_TC || !m.has_chain || m.chain.first_slot != -1 || m.batch != 1) continue;
    const bool row = e.desc.kclass == KB200_K_ROW && (e.impl == IMPL_ROW_LAYERNORM || e.impl == IMPL_ROW_SOFTMAX) && e.row_pre.n >= 1;
    if (!row && (e.desc.kclass != KB200_K_ELEMENTWISE || e.impl == IMPL_FUSED_AWAY || !e.has_chain || e.chain.first_slot < 0)) continue;
    const Chain e_chain = row ? e.row_pre : e.chain;
    const int e_out_slot = row ? e.pre_out_slot : e.chain.out_slot;      // a row kernel need not store the chain's value
    if (numel_of(e.desc) != m.M * m.N || m.chain.n + e_chain.n > kMaxChain) continue;
    if (m.desc.operands[m.chain.out_slot].base_kind != KB200_BASE_ARENA) continue;   // a plan output must be written
    if (!row) {
      std::vector<int> reads, writes;
      reads_and_writes(e, &reads, &writes);
      if (writes.size() != 1) continue;
    }
    const DevOperand mo = m.ops[m.chain.out_slot];
    if (mo.stride[2] != 1 || mo.stride[1] != m.N) continue;
    const Span mo_span = span_of(m, m.chain.out_slot);
    // An operand of the elementwise kernel as a function of the matmul's (row, column): element
    // `delta` of the flat iteration space is row delta / N, column delta % N.
    const kb200_kernel_desc& ed = e.desc;
    auto offset_of = [&](const DevOperand& o, int64_t delta) {
      int64_t off = 0;
      for (int d = ed.iter_rank - 1; d >= 0; --d) {
        off += (delta % ed.iter_shape[d]) * o.stride[d];
        delta /= ed.iter_shape[d];
      }
      return off;
    };
    auto linear = [&](const DevOperand& o, int64_t* s_m, int64_t* s_n) {
      *s_n = m.N > 1 ? offset_of(o, 1) : 0;
      *s_m = m.M > 1 ? offset_of(o, m.N) : 0;
      // every iteration dim must then agree with (s_m, s_n): a dim inside a row, a dim of whole rows, or
      // one that runs across row ends (contiguous dims the host collapsed into one)
      int64_t inner = 1;
      for (int d = ed.iter_rank - 1; d >= 0; --d) {
        const int64_t sh = ed.iter_shape[d], st = o.stride[d];
        if (sh > 1) {
          if (inner >= m.N) {
            if (inner % m.N || st != inner / m.N * *s_m) return false;
          } else if (inner * sh <= m.N) {
            if (m.N % (inner * sh) || st != inner * *s_n) return false;
          } else {
            if (m.N % inner || (inner * sh) % m.N || st != inner * *s_n || *s_m != m.N / inner * st) return false;
          }
        }
        inner *= sh;
      }
      return true;
    };
    auto is_matmul_output = [&](int slot) {
      int64_t s_m, s_n;
      return e.ops[slot].ptr == mo.ptr && linear(e.ops[slot], &s_m, &s_n) && s_n == 1 && s_m == m.N;
    };
    // where the matmul's value enters the elementwise chain: as its first value, or as the other
    // argument of its first step
    Chain tail = e_chain;
    const int acc_slot = is_matmul_output(tail.first_slot) ? tail.first_slot : (tail.n >= 1 ? tail.steps[0].slot : -1);
    if (!is_matmul_output(tail.first_slot)) {
      if (tail.n < 1 || tail.steps[0].slot < 0 || !is_matmul_output(tail.steps[0].slot)) continue;
      int swapped;
      switch (tail.steps[0].op) {
        case CH_ADD: case CH_MUL: case CH_MAX: case CH_MIN: swapped = tail.steps[0].op; break;
        case CH_SUB: swapped = CH_RSUB; break;
        case CH_RSUB: swapped = CH_SUB; break;
        case CH_DIV: swapped = CH_RDIV; break;
        case CH_RDIV: swapped = CH_DIV; break;
        default: swapped = -1; break;
      }
      if (swapped < 0) continue;
      tail.steps[0].op = swapped;
      tail.steps[0].slot = tail.first_slot;
    }
    bool ok = true;
    for (int s = 0; s < tail.n; ++s)
      if (tail.steps[s].slot >= 0 && spans_overlap(span_of(e, tail.steps[s].slot), mo_span)) ok = false;   // reads it a second time
    // nobody else reads the matmul's output before it is rewritten
    bool rewritten = false;
    for (size_t i = j + 2; i < plan.kernels.size() && ok && !rewritten; ++i) {
      const PlanKernel& k = plan.kernels[i];
      if (k.impl == IMPL_FUSED_AWAY && k.absorbed_by < 0) {
        // folded copies read nothing; kernels the fused attention covers stand for its reads and writes
        bool covered = false;
        for (size_t back = 1; back <= 6 && back <= i && !covered; ++back)
          covered = plan.kernels[i - back].impl == IMPL_ATTN_FUSED && (int)back < attention_chain_length(plan.kernels[i - back]);
        if (!covered) continue;
      } else if (k.impl == IMPL_FUSED_AWAY) {
        continue;
      }
      std::vector<int> reads, writes;
      reads_and_writes(k, &reads, &writes);
      for (int slot : reads) ok = ok && !spans_overlap(span_of(k, slot), mo_span);
      for (int slot : writes) {
        const Span w = span_of(k, slot);
        if (w.lo <= mo_span.lo && w.hi >= mo_span.hi) rewritten = true;
        else if (spans_overlap(w, mo_span)) ok = false;
      }
    }
    if (!ok) continue;
    // the new chain, its side operands in fresh slots of the matmul
    PlanKernel merged = m;
    int64_t s_m, s_n;
    for (int s = 0; s < tail.n && ok; ++s) {
      ChainStep step = tail.steps[s];
      if (step.slot >= 0) {
        const DevOperand& o = e.ops[step.slot];
        if (merged.n_ops >= KB200_MAX_OPERANDS || !linear(o, &s_m, &s_n)) { ok = false; break; }
        DevOperand side{};
        side.ptr = o.ptr;
        side.stride[1] = s_m;
        side.stride[2] = s_n;
        step.slot = merged.n_ops;
        merged.ops[merged.n_ops++] = side;
      }
      merged.chain.steps[merged.chain.n++] = step;
    }
    if (!ok || (e_out_slot >= 0 && !linear(e.ops[e_out_slot], &s_m, &s_n))) continue;
    // While the matmul runs its operands are still being read: its output may coincide with a side
    // operand element for element (an add in place), and must not touch anything else the kernel reads.
    auto output_is_safe = [&](const PlanKernel& cand) {
      const DevOperand& o = cand.ops[cand.chain.out_slot];
      const Span o_span = span_of(cand, cand.chain.out_slot);
      std::vector<int> reads, writes;
      reads_and_writes(cand, &reads, &writes);
      for (int slot : reads) {
        const DevOperand& r = cand.ops[slot];
        const bool same = slot >= m.desc.n_operands && r.ptr == o.ptr && r.stride[1] == o.stride[1] && r.stride[2] == o.stride[2];
        if (!same && spans_overlap(span_of(cand, slot), o_span)) return false;
      }
      return true;
    };
    if (row) {
      // the chain's value goes to the row kernel's second output, or stays in the matmul's own buffer;
      // the row kernel reads it there and runs its reductions only
      PlanKernel cand = merged;
      if (e_out_slot >= 0) {
        DevOperand out{};
        out.ptr = e.ops[e_out_slot].ptr;
        out.stride[1] = s_m;
        out.stride[2] = s_n;
        cand.ops[cand.chain.out_slot] = out;
      }
      if (acc_slot < 0 || !output_is_safe(cand) || !tc_eligible(cand)) continue;
      m = cand;
      e.x_slot = e_out_slot >= 0 ? e_out_slot : acc_slot;
      e.row_pre.n = 0;
      e.pre_out_slot = -1;
      continue;
    }
    // (a) the matmul writes the elementwise kernel's output where the plan put it
    PlanKernel direct = merged;
    DevOperand out{};
    out.ptr = e.ops[e_out_slot].ptr;
    out.stride[1] = s_m;
    out.stride[2] = s_n;
    direct.ops[direct.chain.out_slot] = out;
    if (output_is_safe(direct) && tc_eligible(direct)) {
      m = direct;
      e.impl = IMPL_FUSED_AWAY;
      e.launches = 0;
      e.absorbed_by = (int)j;
      continue;
    }
    // (b) the planner reused memory the matmul still reads (its A operand, typically) for that output:
    // the value stays in the matmul's own output buffer instead, and the kernels that read the
    // elementwise kernel's output read it there.  Needs the same layout in both buffers, every such
    // reader inside that output, and the matmul's buffer untouched for as long as the value is live.
    const DevOperand eo = e.ops[e_out_slot];
    if (e.desc.operands[e_out_slot].base_kind != KB200_BASE_ARENA || s_n != 1 || s_m != m.N || (mo.ptr - eo.ptr) % 32 != 0) continue;
    if (!output_is_safe(merged) || !tc_eligible(merged)) continue;
    const Span eo_span = span_of(e, e_out_slot);
    std::vector<std::pair<size_t, int>> redirect;
    bool dead = false;
    for (size_t i = j + 2; i < plan.kernels.size() && ok && !dead; ++i) {
      const PlanKernel& k = plan.kernels[i];
      if (k.impl == IMPL_FUSED_AWAY && k.absorbed_by >= 0) continue;
      if (k.impl == IMPL_ATTN_FUSED) { ok = false; break; }      // its operand pointers are already bound
      if (k.impl == IMPL_FUSED_AWAY) continue;                   // a folded copy
      std::vector<int> reads, writes;
      reads_and_writes(k, &reads, &writes);
      for (int slot : reads) {
        const Span x = span_of(k, slot);
        if (!spans_overlap(x, eo_span)) continue;
        if (x.lo >= eo_span.lo && x.hi <= eo_span.hi) redirect.push_back({i, slot});
        else ok = false;
      }
      for (int slot : writes) {
        const Span x = span_of(k, slot);
        if (spans_overlap(x, mo_span)) ok = false;
        if (x.lo <= eo_span.lo && x.hi >= eo_span.hi) dead = true;
        else if (spans_overlap(x, eo_span)) ok = false;
      }
    }
    if (!ok) continue;
    m = merged;
    for (auto& [i, slot] : redirect) plan.kernels[i].ops[slot].ptr += mo.ptr - eo.ptr;
    e.impl = IMPL_FUSED_AWAY;
    e.launches = 0;
    e.absorbed_by = (int)j;
  }
}

// For every BF16 tensor-core matmul operand that lives in the arena: if the last kernel that wrote
// that memory covers it completely and can also emit bf16, let it write the bf16 mirror and let the
// matmul read the mirror.  Anything else keeps the per-launch conversion pass.
static int assign_shadows(Plan& plan) {
  const float* arena_lo = plan.arena;
  const float* arena_hi = plan.arena + plan.arena_bytes / 4;
  bool any = false;
  // The latest kernel before `ki` that writes into the span x: returned when it is one that can also
  // emit bf16 (LayerNorm, tensor-core matmul, fused attention) and its output covers x inside the arena.
  auto mirroring_producer = [&](size_t ki, const Span& x) -> PlanKernel* {
    for (size_t j = ki; j-- > 0;) {
      PlanKernel& pj = plan.kernels[j];
      if (pj.impl == IMPL_FUSED_AWAY) continue;
      const DevOperand* out = nullptr;
      int64_t out_elems = 0;
      if (pj.impl == IMPL_ATTN_FUSED) {
        out = attention_output(plan, j, &out_elems);
      } else if (pj.impl == IMPL_ROW_LAYERNORM && pj.desc.iter_rank == 2) {
        out = &pj.ops[pj.out_slot];
        out_elems = (pj.desc.iter_shape[0] - 1) * out->stride[0] + pj.desc.iter_shape[1];
      } else if (pj.impl == IMPL_MM_TC && pj.has_chain) {
        out = &pj.ops[pj.chain.out_slot];
        out_elems = (pj.batch - 1) * out->stride[0] + (pj.M - 1) * out->stride[1] + (pj.N - 1) * out->stride[2] + 1;
      } else {
        // some other kernel: does it write into the operand at all?
        bool writes = false;
        for (int t = 0; t < pj.desc.n_tape; ++t)
          if (pj.desc.tape[t].opcode == KB200_OP_STORE) {
            const Span w = span_of(pj, pj.desc.tape[t].b);
            writes = writes || (w.lo < x.hi && x.lo < w.hi);
          }
        if (writes) return nullptr;      // written by a kernel that cannot emit bf16: keep the conversion pass
        continue;
      }
      const Span w{out->ptr, out->ptr + out_elems};
      if (!(w.lo < x.hi && x.lo < w.hi)) continue;                 // does not touch the operand
      if (w.lo <= x.lo && w.hi >= x.hi && w.lo >= arena_lo && w.hi <= arena_hi) return &pj;
      return nullptr;
    }
    return nullptr;
  };
  std::vector<size_t> attention_readers;
  for (size_t ki = 0; ki < plan.kernels.size(); ++ki) {
    PlanKernel& k = plan.kernels[ki];
    if (k.impl == IMPL_ATTN_FUSED && attention_wants_bf16(k)) {
      // the fused attention reads Q, K and V (views of one projection's output) as bf16 when that
      // projection can write them so
      Span x{nullptr, nullptr};
      if (attention_operand_span(k, &x.lo, &x.hi) && x.lo >= arena_lo && x.hi <= arena_hi && (x.lo - arena_lo) % 8 == 0) {
        if (PlanKernel* pj = mirroring_producer(ki, x)) {
          pj->shadow_out = reinterpret_cast<void*>(1);
          attention_readers.push_back(ki);
          any = true;
        }
      }
      continue;
    }
    if (k.impl != IMPL_MM_TC || !matmul_wants_bf16_operands(k)) continue;
    for (int role = 0; role < 2; ++role) {
      const int slot = role == 0 ? k.desc.a_slot : k.desc.b_slot;
      if (k.desc.operands[slot].base_kind != KB200_BASE_ARENA) continue;
      const Span x = span_of(k, slot);
      if (x.lo < arena_lo || x.hi > arena_hi) continue;
      // the mirror is read through TMA: 16-byte aligned base and strides in 2-byte elements
      const DevOperand& xo = k.ops[slot];
      if ((x.lo - arena_lo) % 8 || xo.stride[0] % 8 || xo.stride[1] % 8 || xo.stride[2] % 8 && xo.stride[2] != 1) continue;
      if (PlanKernel* pj = mirroring_producer(ki, x)) {
        pj->shadow_out = reinterpret_cast<void*>(1);                // marked; the address is filled in below
        (role == 0 ? k.a_shadow : k.b_shadow) = reinterpret_cast<const void*>(1);
        any = true;
      }
    }
  }
  if (!any) return KB200_OK;
  const uint64_t need = plan.arena_bytes / 2 + 256;
  if (plan.arena16 == nullptr || plan.arena16_bytes < need) {
    if (plan.arena16) cudaFree(plan.arena16);
    plan.arena16 = nullptr;
    KB200_CUDA(cudaMalloc(&plan.arena16, need));
    plan.arena16_bytes = need;
  }
  uint16_t* mirror = static_cast<uint16_t*>(plan.arena16);
  auto mirror_of = [&](const float* ptr) { return static_cast<void*>(mirror + (ptr - plan.arena)); };
  for (size_t ki = 0; ki < plan.kernels.size(); ++ki) {
    PlanKernel& k = plan.kernels[ki];
    if (k.shadow_out) {
      const DevOperand* out;
      int64_t elems;
      if (k.impl == IMPL_ATTN_FUSED) out = attention_output(plan, ki, &elems);
      else if (k.impl == IMPL_ROW_LAYERNORM) out = &k.ops[k.out_slot];
      else out = &k.ops[k.chain.out_slot];
      k.shadow_out = mirror_of(out->ptr);
      if (k.impl == IMPL_ATTN_FUSED) attention_set_shadow(k, k.shadow_out);
    }
    if (k.a_shadow) k.a_shadow = mirror_of(k.ops[k.desc.a_slot].ptr);
    if (k.b_shadow) k.b_shadow = mirror_of(k.ops[k.desc.b_slot].ptr);
  }
  for (size_t ki : attention_readers) attention_use_mirror(plan.kernels[ki], plan.arena, plan.arena16);
  if (!plan.mirror_only) return KB200_OK;
  // A LayerNorm or matmul that writes the mirror drops its float32 store when, until that memory is
  // rewritten (or the plan ends: arena contents are dead then), every reader takes the mirror.
  for (size_t ki = 0; ki < plan.kernels.size(); ++ki) {
    PlanKernel& k = plan.kernels[ki];
    if (!k.shadow_out || (k.impl != IMPL_ROW_LAYERNORM && k.impl != IMPL_MM_TC)) continue;
    const int out_slot = k.impl == IMPL_ROW_LAYERNORM ? k.out_slot : k.chain.out_slot;
    const Span w = span_of(k, out_slot);
    bool only = true, rewritten = false;
    int readers = 0;
    for (size_t i = ki + 1; i < plan.kernels.size() && only && !rewritten; ++i) {
      const PlanKernel& r = plan.kernels[i];
      if (r.impl == IMPL_FUSED_AWAY) continue;     // folded, absorbed, or stood for by the fused attention's own kernel
      if (r.impl == IMPL_ATTN_FUSED) {
        Span x{nullptr, nullptr};
        if (!attention_operand_span(r, &x.lo, &x.hi)) { only = false; break; }
        if (spans_overlap(x, w)) {
          if (attention_reads_mirror(r) && w.lo <= x.lo && w.hi >= x.hi) ++readers;
          else only = false;
        }
        int64_t elems = 0;
        const DevOperand* y = attention_output(plan, i, &elems);
        const Span yw{y->ptr, y->ptr + elems};
        if (yw.lo <= w.lo && yw.hi >= w.hi) rewritten = true;
        else if (spans_overlap(yw, w)) only = false;
        continue;
      }
      std::vector<int> reads, writes;
      reads_and_writes(r, &reads, &writes);
      for (int slot : reads) {
        const Span x = span_of(r, slot);
        if (!spans_overlap(x, w)) continue;
        const bool mirrored = r.impl == IMPL_MM_TC && ((slot == r.desc.a_slot && r.a_shadow) || (slot == r.desc.b_slot && r.b_shadow));
        if (mirrored && w.lo <= x.lo && w.hi >= x.hi) ++readers;
        else only = false;
      }
      for (int slot : writes) {
        const Span x = span_of(r, slot);
        if (x.lo <= w.lo && x.hi >= w.hi) rewritten = true;
        else if (spans_overlap(x, w)) only = false;
      }
    }
    k.mirror_only = only && readers > 0;
  }
  return KB200_OK;
}

static int launch_one(const Plan& plan, const PlanKernel& k, cudaStream_t s) {
  if (numel_of(k.desc) == 0 || k.impl == IMPL_FUSED_AWAY) return KB200_OK;
  if (k.impl == IMPL_ATTN_FUSED) return attention_launch(plan, k, s);
  switch (k.desc.kclass) {
    case KB200_K_ELEMENTWISE: return launch_elementwise(plan, k, s);
    case KB200_K_ROW: return launch_row(plan, k, s);
    case KB200_K_REDUCE: return launch_reduce(plan, k, s);
    default: return launch_matmul(plan, k, s);
  }
}

}  // namespace kb200

using namespace kb200;

KB200_EXPORT int kb200_version(void) { return KB200_ABI_VERSION; }

KB200_EXPORT const char* kb200_last_error(void) { return g_error.c_str(); }

KB200_EXPORT int kb200_plan_create(const kb200_kernel_desc* descs, int n, int device, kb200_plan** out) {
  if (out == nullptr) return fail(KB200_ERR_ARGUMENT, "kb200_plan_create: out is null");
  *out = nullptr;
  if (n < 0 || (n > 0 && descs == nullptr)) return fail(KB200_ERR_ARGUMENT, "kb200_plan_create: bad descriptor array");
  int count = 0;
  KB200_CUDA(cudaGetDeviceCount(&count));
  if (device < 0 || device >= count) return fail(KB200_ERR_ARGUMENT, "kb200_plan_create: no CUDA device %d", device);
  cudaDeviceProp prop;
  KB200_CUDA(cudaGetDeviceProperties(&prop, device));
  if (prop.major != 10)
    return fail(KB200_ERR_UNSUPPORTED, "kb200_plan_create: device %d is sm_%d%d; this library is built for sm_100a only",
                device, prop.major, prop.minor);
  for (int i = 0; i < n; ++i) {
    int rc = validate(descs[i], i);
    if (rc) return rc;
  }
  Plan* plan = new (std::nothrow) Plan();
  if (!plan) return fail(KB200_ERR_ARGUMENT, "kb200_plan_create: out of host memory");
  plan->device = device;
  plan->sm_count = prop.multiProcessorCount;
  plan->kernels.resize(n);
  for (int i = 0; i < n; ++i) {
    PlanKernel& k = plan->kernels[i];
    k.desc = descs[i];
    k.desc.name[sizeof(k.desc.name) - 1] = 0;
    k.tape.n = descs[i].n_tape;
    memcpy(k.tape.ops, descs[i].tape, sizeof(kb200_tape_op) * descs[i].n_tape);
    if (k.desc.kclass == KB200_K_MATMUL) {
      k.batch = k.desc.iter_shape[0];
      k.M = k.desc.iter_shape[1];
      k.N = k.desc.iter_shape[2];
      k.K = k.desc.k_extent;
    }
  }
  int prev = 0;
  cudaGetDevice(&prev);
  cudaError_t e = cudaSetDevice(device);
  if (e == cudaSuccess) e = cudaMalloc(&plan->d_status, sizeof(int));
  if (e == cudaSuccess) e = cudaMemset(plan->d_status, 0, sizeof(int));
  cudaSetDevice(prev);
  if (e != cudaSuccess) {
    delete plan;
    return cuda_fail(e, "allocating the plan's status word");
  }
  *out = reinterpret_cast<kb200_plan*>(plan);
  return KB200_OK;
}

KB200_EXPORT int kb200_plan_bind(kb200_plan* p, void* arena, uint64_t arena_bytes, void* const* consts,
                                 const uint64_t* const_bytes, int n_consts, void* const* inputs,
                                 const uint64_t* input_bytes, int n_inputs, void* const* outputs,
                                 const uint64_t* output_bytes, int n_outputs) {
  if (p == nullptr) return fail(KB200_ERR_ARGUMENT, "kb200_plan_bind: plan is null");
  Plan& plan = *reinterpret_cast<Plan*>(p);
  if (n_consts < 0 || n_inputs < 0 || n_outputs < 0 || (n_consts && (!consts || !const_bytes)) ||
      (n_inputs && (!inputs || !input_bytes)) || (n_outputs && (!outputs || !output_bytes)))
    return fail(KB200_ERR_ARGUMENT, "kb200_plan_bind: bad buffer arrays");
  plan.bound = false;
  plan.arena = static_cast<float*>(arena);
  plan.arena_bytes = arena_bytes;
  auto fill = [](std::vector<float*>& ptrs, std::vector<uint64_t>& sizes, void* const* src, const uint64_t* bytes, int n) {
    ptrs.resize(n);
    sizes.resize(n);
    for (int i = 0; i < n; ++i) { ptrs[i] = static_cast<float*>(src[i]); sizes[i] = bytes[i]; }
  };
  fill(plan.consts, plan.const_bytes, consts, const_bytes, n_consts);
  fill(plan.inputs, plan.input_bytes, inputs, input_bytes, n_inputs);
  fill(plan.outputs, plan.output_bytes, outputs, output_bytes, n_outputs);
  int prev = 0;
  cudaGetDevice(&prev);
  KB200_CUDA(cudaSetDevice(plan.device));
  int rc = KB200_OK;
  // phase 1: resolve pointers, pick an implementation per kernel
  for (size_t i = 0; i < plan.kernels.size() && rc == KB200_OK; ++i) {
    PlanKernel& k = plan.kernels[i];
    attention_destroy(k);
    k.shadow_out = nullptr;
    k.a_shadow = k.b_shadow = nullptr;
    k.mirror_only = false;
    k.absorbed_by = -1;
    k.n_ops = k.desc.n_operands;
    rc = resolve(plan, k, (int)i);
    if (rc) break;
    switch (k.desc.kclass) {
      case KB200_K_ELEMENTWISE: rc = choose_elementwise(plan, k); break;
      case KB200_K_ROW: rc = choose_row(plan, k); break;
      case KB200_K_REDUCE: rc = choose_reduce(plan, k); break;
      default: rc = choose_matmul(plan, k); break;
    }
  }
  // phase 2: fuse the attention chain where it matches
  if (rc == KB200_OK && plan.fuse_attention)
    for (size_t i = 0; i + 4 < plan.kernels.size(); ++i) {
      const int fused = attention_try_fuse(plan, i);
      if (fused > 0) i += fused - 1;
    }
  // phase 2b: matmuls read a K-contiguous B at its source instead of through the plan's transposing copy
  if (rc == KB200_OK && plan.fold_copies) fold_operand_copies(plan);
  // phase 2c: a tensor-core matmul also runs the elementwise kernel that only continues it
  if (rc == KB200_OK && plan.absorb_elementwise) absorb_elementwise(plan);
  // phase 3: BF16 matmuls read activations from the bf16 mirror when their producer can write it
  if (rc == KB200_OK) rc = assign_shadows(plan);
  for (size_t i = 0; i < plan.kernels.size() && rc == KB200_OK; ++i)
    if (plan.kernels[i].impl == IMPL_ATTN_FUSED) attention_elide_copy(plan, i);
  // phase 4: tensor maps, packed weights, split-K workspaces
  for (size_t i = 0; i < plan.kernels.size() && rc == KB200_OK; ++i) {
    PlanKernel& k = plan.kernels[i];
    if (k.desc.kclass == KB200_K_MATMUL && k.impl != IMPL_FUSED_AWAY) rc = bind_matmul(plan, k);
  }
  cudaSetDevice(prev);
  if (rc) return rc;
  plan.bound = true;
  return KB200_OK;
}

KB200_EXPORT int kb200_plan_set_option(kb200_plan* p, int option, int value) {
  if (p == nullptr) return fail(KB200_ERR_ARGUMENT, "kb200_plan_set_option: plan is null");
  Plan& plan = *reinterpret_cast<Plan*>(p);
  switch (option) {
    case KB200_OPT_FUSE_ATTENTION: plan.fuse_attention = value != 0; return KB200_OK;
    case KB200_OPT_DEPENDENT_LAUNCH: plan.pdl = value != 0; return KB200_OK;
    case KB200_OPT_FOLD_OPERAND_COPIES: plan.fold_copies = value != 0; return KB200_OK;
    case KB200_OPT_CONCURRENCY: plan.concurrency = value < 1 ? 1 : value; return KB200_OK;
    case KB200_OPT_ABSORB_ELEMENTWISE: plan.absorb_elementwise = value != 0; return KB200_OK;
    case KB200_OPT_MIRROR_ONLY: plan.mirror_only = value != 0; return KB200_OK;
    case KB200_OPT_FP32_ATTENTION: plan.fp32_attention = value < 0 || value > 2 ? 0 : value; return KB200_OK;
    case KB200_OPT_ATTENTION_SPLIT: plan.attention_split = value != 0; return KB200_OK;
    default: return fail(KB200_ERR_ARGUMENT, "kb200_plan_set_option: unknown option %d", option);
  }
}

KB200_EXPORT int kb200_plan_launch(kb200_plan* p, void* stream) {
  if (p == nullptr) return fail(KB200_ERR_ARGUMENT, "kb200_plan_launch: plan is null");
  Plan& plan = *reinterpret_cast<Plan*>(p);
  if (!plan.bound) return fail(KB200_ERR_UNBOUND, "kb200_plan_launch: call kb200_plan_bind first");
  for (size_t i = 0; i < plan.kernels.size(); ++i) {
    int rc = launch_one(plan, plan.kernels[i], static_cast<cudaStream_t>(stream));
    if (rc) return rc;
  }
  return KB200_OK;
}

KB200_EXPORT int kb200_kernel_launch(kb200_plan* p, int i, void* stream) {
  if (p == nullptr) return fail(KB200_ERR_ARGUMENT, "kb200_kernel_launch: plan is null");
  Plan& plan = *reinterpret_cast<Plan*>(p);
  if (!plan.bound) return fail(KB200_ERR_UNBOUND, "kb200_kernel_launch: call kb200_plan_bind first");
  if (i < 0 || i >= (int)plan.kernels.size()) return fail(KB200_ERR_ARGUMENT, "kb200_kernel_launch: no kernel %d", i);
  return launch_one(plan, plan.kernels[i], static_cast<cudaStream_t>(stream));
}

KB200_EXPORT int kb200_plan_launch_count(const kb200_plan* p) {
  if (p == nullptr) return 0;
  const Plan& plan = *reinterpret_cast<const Plan*>(p);
  int n = 0;
  for (const PlanKernel& k : plan.kernels) n += numel_of(k.desc) == 0 ? 0 : k.launches;
  return n;
}

KB200_EXPORT const char* kb200_kernel_impl(const kb200_plan* p, int i) {
  if (p == nullptr) return "?";
  const Plan& plan = *reinterpret_cast<const Plan*>(p);
  if (i < 0 || i >= (int)plan.kernels.size()) return "?";
  if (!plan.bound) return "unbound";
  return impl_name(plan.kernels[i].impl);
}

KB200_EXPORT int kb200_kernel_chain_length(const kb200_plan* p, int i) {
  if (p == nullptr) return -1;
  const Plan& plan = *reinterpret_cast<const Plan*>(p);
  if (i < 0 || i >= (int)plan.kernels.size() || !plan.bound) return -1;
  const PlanKernel& k = plan.kernels[i];
  switch (k.impl) {
    case IMPL_MM_TC: case IMPL_MM_GEMV: case IMPL_MM_SIMT: case IMPL_EW_CHAIN_VEC4: case IMPL_EW_TRANSPOSE:
      return k.has_chain ? k.chain.n : 0;
    case IMPL_ROW_LAYERNORM: case IMPL_ROW_SOFTMAX: return k.row_pre.n;
    default: return 0;
  }
}

KB200_EXPORT int kb200_plan_status(kb200_plan* p) {
  if (p == nullptr) return fail(KB200_ERR_ARGUMENT, "kb200_plan_status: plan is null");
  Plan& plan = *reinterpret_cast<Plan*>(p);
  int word = 0;
  KB200_CUDA(cudaMemcpy(&word, plan.d_status, sizeof(int), cudaMemcpyDeviceToHost));
  if (word != 0) {
    cudaMemset(plan.d_status, 0, sizeof(int));
    // a fused attention that gave up may have counted one half of a shared query tile and not the other
    for (PlanKernel& k : plan.kernels) attention_reset_arrivals(k);
    return fail(KB200_ERR_DEVICE_WAIT, "a bounded device-side wait ran out (code 0x%x: kernel %d, site %d)", word,
                (word >> 8) & 0xffff, word & 0xff);
  }
  return KB200_OK;
}

// ---------------------------------------------------------------------------------------------
// Failure-path self-test: a wait that is MEANT to run out, in the only safe form -- one warp, one
// mbarrier that expects two arrivals and gets one, no copy in flight, a few thousand polls.  The
// kernel then does what the tensor-core kernels do when a wait expires: records (kernel, site) in the
// plan's status word and returns normally, so the context stays usable and kb200_plan_status reports
// KB200_ERR_DEVICE_WAIT.
// ---------------------------------------------------------------------------------------------
namespace kb200 {
namespace {
__global__ void expiring_wait_kernel(int* status, int polls) {
  __shared__ __align__(8) uint64_t bar;
  const uint32_t addr = (uint32_t)__cvta_generic_to_shared(&bar);
  if (threadIdx.x == 0) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(addr), "r"(2));
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(addr) : "memory");   // one of the two arrivals
    bool done = false;
    for (int i = 0; i < polls && !done; ++i) {
      uint32_t ok;
      asm volatile("{\n\t.reg .pred p;\n\tmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                   : "=r"(ok) : "r"(addr), "r"(0) : "memory");
      done = ok != 0;
    }
    if (!done) atomicCAS(status, 0, (0xFFFF << 8) | 0x7F);
    asm volatile("mbarrier.inval.shared::cta.b64 [%0];" ::"r"(addr) : "memory");
  }
}
}  // namespace
}  // namespace kb200

KB200_EXPORT int kb200_plan_selftest_wait(kb200_plan* p, void* stream) {
  if (p == nullptr) return fail(KB200_ERR_ARGUMENT, "kb200_plan_selftest_wait: plan is null");
  Plan& plan = *reinterpret_cast<Plan*>(p);
  expiring_wait_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(plan.d_status, 4096);
  KB200_CUDA(cudaGetLastError());
  return KB200_OK;
}

KB200_EXPORT void kb200_plan_destroy(kb200_plan* p) {
  if (p == nullptr) return;
  Plan* plan = reinterpret_cast<Plan*>(p);
  int prev = 0;
  cudaGetDevice(&prev);
  cudaSetDevice(plan->device);
  for (PlanKernel& k : plan->kernels) {
    destroy_matmul(k);
    attention_destroy(k);
  }
  if (plan->d_status) cudaFree(plan->d_status);
  if (plan->arena16) cudaFree(plan->arena16);
  cudaSetDevice(prev);
  delete plan;
}
