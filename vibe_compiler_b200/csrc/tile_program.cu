// Replay of the per-Tile target LLVM modules the reference compiler emits: a text parser and interpreter for the
// closed integer IR subset the reference admits for host execution
// (lib/Wafer/Simulator/Invocation/TargetCallExecution.cpp:188-294), a cooperative scheduler over the Tiles with the
// Direct-DTE matching rule of lib/Wafer/Simulator/SystemC/SystemCTargetModel.cpp:1110-1200, an address plan built from
// the !wafer.target.entry_arguments rows (lib/Wafer/CodeGen/LLVM/TargetLLVMTranslation.cpp:119-140), and the routing
// of every wafer_tx81_* call to the device executors. Host logic only; the kernels live in tile_movement.cu,
// gemm_formal.cu and gemm_umma.cu.
#include <ctype.h>
#include <stdlib.h>

#include <algorithm>
#include <map>
#include <memory>
#include <string>
#include <utility>
#include <vector>

#include "backend.h"

namespace wb200 {
namespace {

// ------------------------------------------------------------------------------------------------ IR model
enum class Op : uint8_t {
  Add, Sub, Mul, UDiv, SDiv, URem, SRem, And, Or, Xor, Shl, LShr, AShr,
  ICmp, Phi, Select, ZExt, SExt, Trunc, Freeze, SMin, SMax, UMin, UMax, Call, Br, CondBr, Switch, Ret
};
enum class Pred : uint8_t { Eq, Ne, Ugt, Uge, Ult, Ule, Sgt, Sge, Slt, Sle };

struct Operand {
  bool is_constant = true;
  uint64_t constant = 0;
  int reg = -1;
};

struct Inst {
  Op op = Op::Ret;
  Pred pred = Pred::Eq;
  int dst = -1;
  int bits = 64;       // result width (operand width for icmp and casts' source in src_bits)
  int src_bits = 64;
  Operand a, b, c;
  std::vector<std::pair<Operand, std::string>> incoming_names;  // phi, before label resolution
  std::vector<std::pair<Operand, int>> incoming;                // phi
  std::vector<std::pair<uint64_t, std::string>> case_names;     // switch
  std::vector<std::pair<uint64_t, int>> cases;
  std::string target_names[2];
  int targets[2] = {-1, -1};
  int command = -1;    // Call: index into kCommands
  uint32_t operation = 0;   // Call: elementwise operation / convert opcode of the symbol-selected families
  std::vector<Operand> args;
};

struct Block {
  std::string label;
  std::vector<Inst> insts;
  size_t first_non_phi = 0;
};

struct MetaField {
  bool is_string = false;
  int64_t integer = 0;
  std::string text;
  int node = -1;       // reference to another node (!N)
};

struct EntrySlot {
  int64_t ordinal = 0;
  std::string kind, name, format, layout, access;
  int64_t resource = 0, bytes = 0, alignment = 1, zero_initialize = 0;
  std::vector<int64_t> shape;
  uint64_t address = 0;   // assigned by the address plan
};

struct Module {
  int tile_id = -1;
  int arg_count = 0;
  int reg_count = 0;
  std::vector<Block> blocks;
  std::vector<EntrySlot> slots;
};

// ------------------------------------------------------------------------------------------------ commands
enum Command : int {
  kNccJoin, kDteBegin, kDteBeginAfterPrepare, kDteSendPrepare, kDteSendIssue, kDteRecvPrepare, kDteWait, kDteFinish,
  kRdma, kWdma, kGatherScatter, kMemset, kGemm, kGemmOriented,
  // Families whose symbol carries the operation (wafer_tx81_elementwise_<op>, wafer_tx81_convert_<route>):
  kElementwiseUnary, kElementwiseBinary, kElementwiseLogic, kConvert, kReduce, kPool, kBit2Fp, kMaskMove, kCommandCount
};
struct CommandInfo {
  const char *symbol;
  int argc;           // including the trailing NCC worker where the ABI has one
  bool has_worker;
  bool returns_value;
};
// Argument counts follow lib/Wafer/Target/TargetCall.cpp:60-147 (i64 addresses first, then i32 fields, then the worker).
const CommandInfo kCommands[kCommandCount] = {
    {"wafer_tx81_ncc_join", 1, false, false},
    {"wafer_tx81_direct_dte_begin", 2, false, false},
    {"wafer_tx81_direct_dte_begin_after_prepare", 2, false, false},
    {"wafer_tx81_direct_dte_send_prepare", 7, false, true},
    {"wafer_tx81_direct_dte_send_issue", 1, false, false},
    {"wafer_tx81_direct_dte_recv_prepare", 5, false, true},
    {"wafer_tx81_direct_dte_wait", 1, false, false},
    {"wafer_tx81_direct_dte_finish", 0, false, false},
    {"wafer_tx81_rdma", 12, true, false},
    {"wafer_tx81_wdma", 12, true, false},
    {"wafer_tx81_gather_scatter", 17, true, false},
    {"wafer_tx81_memset", 5, true, false},
    {"wafer_tx81_gemm", 12, true, false},
    {"wafer_tx81_gemm_oriented", 14, true, false},
    {"wafer_tx81_elementwise_unary", 5, true, false},     // (source, destination; count, format; worker)
    {"wafer_tx81_elementwise_binary", 9, true, false},    // (lhs, rhs | scalar bits, destination; count, format, rhs unit, scalar flag, numeric | rhs group; worker)
    {"wafer_tx81_elementwise_logic", 6, true, false},     // (lhs, rhs, destination; count, format; worker)
    {"wafer_tx81_convert", 6, true, false},               // (source, destination; count, zero point, rounding mode; worker)
    {"wafer_tx81_reduce", 9, true, false},                // (source, destination; dimension, n, h, w, c, format; worker)
    // (input, destination; kind, source nhwc[4], destination nhwc[4], pads[4], kernel w, kernel h, stride w, stride h, format; worker)
    {"wafer_tx81_pool", 21, true, false},
    {"wafer_tx81_bit2fp", 5, true, false},                // (source, destination; count, format; worker)
    {"wafer_tx81_mask_move", 6, true, false},             // (source, mask, destination, count, format; worker)
};

// Spellings of lib/Wafer/Target/TargetOperation.cpp:181-251 in enumeration order (index 11 is unused) and of the convert
// routes 139..174 (lib/Wafer/Target/TargetFormat.cpp:163-200).
const char *const kElementwiseNames[35] = {
    "abs", "recip", "square", "sqrt", "rsqrt", "neg", "max", "min", "add", "sub", "mul", nullptr, "eq", "ne", "ge", "gt", "le", "lt",
    "logic_not", "logic_and", "logic_or", "logic_xor", "log2", "ln", "pow2", "exp", "exp_lp", "sin", "cos", "tanh", "sigmoid", "relu",
    "satrelu", "leakyrelu", "softplus"};
const char *const kConvertNames[36] = {
    "int8_fp16", "int8_bf16", "int8_fp32", "int8_tf32", "int16_fp16", "int16_bf16", "int16_fp32", "int16_tf32", "int32_fp16",
    "int32_bf16", "int32_fp32", "int32_tf32", "bf16_int8", "bf16_int16", "bf16_int32", "bf16_fp16", "bf16_fp32", "bf16_tf32",
    "fp16_int8", "fp16_int16", "fp16_int32", "fp16_bf16", "fp16_fp32", "fp16_tf32", "fp32_int8", "fp32_int16", "fp32_int32",
    "fp32_fp16", "fp32_bf16", "fp32_tf32", "tf32_int8", "tf32_int16", "tf32_int32", "tf32_fp16", "tf32_bf16", "tf32_fp32"};

// -> command index, with *operation = the elementwise operation or the convert opcode for the two families.
int find_command(const std::string &symbol, uint32_t *operation) {
  *operation = 0;
  for (int i = 0; i < kElementwiseUnary; ++i)
    if (symbol == kCommands[i].symbol) return i;
  for (int i = kBit2Fp; i < kCommandCount; ++i)
    if (symbol == kCommands[i].symbol) return i;
  const std::string elementwise = "wafer_tx81_elementwise_", convert = "wafer_tx81_convert_", reduce = "wafer_tx81_reduce_";
  const std::string pool = "wafer_tx81_pool_";
  if (symbol.compare(0, pool.size(), pool) == 0) {   // plain pooling only (lib/Wafer/Target/TargetCall.cpp:113-118); *operation = the target opcode
    const std::string name = symbol.substr(pool.size());
    *operation = name == "sum" ? 116u : name == "max" ? 117u : name == "min" ? 119u : 0u;
    return *operation ? kPool : -1;
  }
  if (symbol.compare(0, reduce.size(), reduce) == 0) {   // lib/Wafer/Target/TargetOperation.cpp stringifyTargetReduceOperation
    const char *const names[4] = {"sum", "max", "min", "avg"};
    for (uint32_t op = 0; op < 4; ++op)
      if (symbol.substr(reduce.size()) == names[op]) {
        *operation = op;
        return kReduce;
      }
    return -1;
  }
  if (symbol.compare(0, elementwise.size(), elementwise) == 0) {
    const std::string name = symbol.substr(elementwise.size());
    for (uint32_t op = 0; op < 35; ++op)
      if (kElementwiseNames[op] && name == kElementwiseNames[op]) {
        *operation = op;
        const bool binary = (op >= WB200_EW_MAX && op <= WB200_EW_LT) || (op >= WB200_EW_LOGIC_AND && op <= WB200_EW_LOGIC_XOR);
        if (!binary) return kElementwiseUnary;
        return op >= WB200_EW_LOGIC_AND ? kElementwiseLogic : kElementwiseBinary;
      }
    return -1;
  }
  if (symbol.compare(0, convert.size(), convert) == 0) {
    const std::string name = symbol.substr(convert.size());
    for (uint32_t route = 0; route < 36; ++route)
      if (name == kConvertNames[route]) {
        *operation = 139 + route;
        return kConvert;
      }
  }
  return -1;
}

// ------------------------------------------------------------------------------------------------ parser
struct Cursor {
  const std::string &s;
  size_t at = 0;
  explicit Cursor(const std::string &text) : s(text) {}
  void skip() { while (at < s.size() && (s[at] == ' ' || s[at] == '\t' || s[at] == ',')) ++at; }
  bool done() { skip(); return at >= s.size(); }
  bool eat(char c) { skip(); if (at < s.size() && s[at] == c) { ++at; return true; } return false; }
  std::string word() {   // identifier-like token: letters, digits, '.', '_', '%', '@', '-', '!'
    skip();
    size_t begin = at;
    while (at < s.size() && (isalnum(static_cast<unsigned char>(s[at])) || s[at] == '.' || s[at] == '_' || s[at] == '%' ||
                             s[at] == '@' || s[at] == '-' || s[at] == '!' || s[at] == '$'))
      ++at;
    return s.substr(begin, at - begin);
  }
  std::string peek_word() { size_t keep = at; std::string w = word(); at = keep; return w; }
};

bool parse_int_type(const std::string &token, int *bits) {
  if (token.size() < 2 || token[0] != 'i') return false;
  for (size_t i = 1; i < token.size(); ++i) if (!isdigit(static_cast<unsigned char>(token[i]))) return false;
  *bits = atoi(token.c_str() + 1);
  return *bits >= 1 && *bits <= 64;
}

uint64_t mask_to(uint64_t value, int bits) { return bits >= 64 ? value : value & ((uint64_t(1) << bits) - 1); }
int64_t sign_extend(uint64_t value, int bits) {
  if (bits >= 64) return static_cast<int64_t>(value);
  const uint64_t sign = uint64_t(1) << (bits - 1);
  value = mask_to(value, bits);
  return static_cast<int64_t>((value ^ sign) - sign);
}

struct ModuleParser {
  Module module;
  std::map<std::string, int> regs;
  std::map<int, std::vector<MetaField>> nodes;
  std::map<std::string, std::vector<MetaField>> named;
  std::string error;

  int reg_of(const std::string &name) {
    auto it = regs.find(name);
    if (it != regs.end()) return it->second;
    const int index = static_cast<int>(regs.size());
    regs[name] = index;
    return index;
  }

  bool operand(Cursor &c, int bits, Operand *out) {
    std::string token = c.word();
    if (token.empty()) { error = "missing operand"; return false; }
    if (token[0] == '%') { out->is_constant = false; out->reg = reg_of(token); return true; }
    out->is_constant = true;
    if (token == "true") { out->constant = 1; return true; }
    if (token == "false" || token == "zeroinitializer") { out->constant = 0; return true; }
    if (token == "undef" || token == "poison") { out->constant = 0; return true; }
    char *end = nullptr;
    const long long value = strtoll(token.c_str(), &end, 10);
    if (*end != '\0') { error = "operand '" + token + "' is not an integer or a value name"; return false; }
    out->constant = mask_to(static_cast<uint64_t>(value), bits);
    return true;
  }

  bool typed_operand(Cursor &c, Operand *out, int *bits_out = nullptr) {
    int bits = 0;
    const std::string type = c.word();
    if (!parse_int_type(type, &bits)) { error = "type '" + type + "' is outside the integer subset"; return false; }
    if (bits_out) *bits_out = bits;
    return operand(c, bits, out);
  }

  bool parse_instruction(const std::string &line, Inst *inst) {
    Cursor c(line);
    std::string first = c.word();
    if (first.empty()) { error = "empty instruction"; return false; }
    if (first[0] == '%') {
      inst->dst = reg_of(first);
      if (!c.eat('=')) { error = "expected '=' after " + first; return false; }
      first = c.word();
    }
    static const std::map<std::string, Op> binary = {
        {"add", Op::Add}, {"sub", Op::Sub}, {"mul", Op::Mul}, {"udiv", Op::UDiv}, {"sdiv", Op::SDiv}, {"urem", Op::URem},
        {"srem", Op::SRem}, {"and", Op::And}, {"or", Op::Or}, {"xor", Op::Xor}, {"shl", Op::Shl}, {"lshr", Op::LShr}, {"ashr", Op::AShr}};
    auto bin = binary.find(first);
    if (bin != binary.end()) {
      inst->op = bin->second;
      std::string type = c.word();
      while (type == "nsw" || type == "nuw" || type == "exact" || type == "disjoint") type = c.word();
      if (!parse_int_type(type, &inst->bits)) { error = "binary operator on non-integer type '" + type + "'"; return false; }
      return operand(c, inst->bits, &inst->a) && operand(c, inst->bits, &inst->b);
    }
    if (first == "icmp") {
      inst->op = Op::ICmp;
      static const std::map<std::string, Pred> preds = {{"eq", Pred::Eq}, {"ne", Pred::Ne}, {"ugt", Pred::Ugt}, {"uge", Pred::Uge},
          {"ult", Pred::Ult}, {"ule", Pred::Ule}, {"sgt", Pred::Sgt}, {"sge", Pred::Sge}, {"slt", Pred::Slt}, {"sle", Pred::Sle}};
      std::string pred = c.word();
      if (pred == "samesign") pred = c.word();
      auto it = preds.find(pred);
      if (it == preds.end()) { error = "unknown icmp predicate '" + pred + "'"; return false; }
      inst->pred = it->second;
      inst->bits = 1;
      if (!parse_int_type(c.word(), &inst->src_bits)) { error = "icmp on a non-integer type"; return false; }
      return operand(c, inst->src_bits, &inst->a) && operand(c, inst->src_bits, &inst->b);
    }
    if (first == "phi") {
      inst->op = Op::Phi;
      if (!parse_int_type(c.word(), &inst->bits)) { error = "phi of a non-integer type"; return false; }
      while (c.eat('[')) {
        Operand value;
        if (!operand(c, inst->bits, &value)) return false;
        const std::string label = c.word();
        if (label.empty() || label[0] != '%' || !c.eat(']')) { error = "malformed phi incoming"; return false; }
        inst->incoming_names.emplace_back(value, label.substr(1));
      }
      if (inst->incoming_names.empty()) { error = "phi without incoming values"; return false; }
      return true;
    }
    if (first == "select") {
      inst->op = Op::Select;
      int cond_bits = 0;
      if (!typed_operand(c, &inst->a, &cond_bits) || cond_bits != 1) { if (error.empty()) error = "select condition must be i1"; return false; }
      return typed_operand(c, &inst->b, &inst->bits) && typed_operand(c, &inst->c);
    }
    if (first == "zext" || first == "sext" || first == "trunc") {
      inst->op = first == "zext" ? Op::ZExt : first == "sext" ? Op::SExt : Op::Trunc;
      std::string type = c.word();
      while (type == "nneg" || type == "nsw" || type == "nuw") type = c.word();
      if (!parse_int_type(type, &inst->src_bits)) { error = "cast from a non-integer type"; return false; }
      if (!operand(c, inst->src_bits, &inst->a)) return false;
      if (c.word() != "to" || !parse_int_type(c.word(), &inst->bits)) { error = "cast to a non-integer type"; return false; }
      return true;
    }
    if (first == "freeze") {
      inst->op = Op::Freeze;
      return typed_operand(c, &inst->a, &inst->bits);
    }
    if (first == "br") {
      std::string token = c.word();
      if (token == "label") {
        inst->op = Op::Br;
        inst->target_names[0] = c.word().substr(1);
        return true;
      }
      int bits = 0;
      if (!parse_int_type(token, &bits) || bits != 1) { error = "conditional branch needs an i1 condition"; return false; }
      inst->op = Op::CondBr;
      if (!operand(c, 1, &inst->a)) return false;
      if (c.word() != "label") { error = "malformed conditional branch"; return false; }
      inst->target_names[0] = c.word().substr(1);
      if (c.word() != "label") { error = "malformed conditional branch"; return false; }
      inst->target_names[1] = c.word().substr(1);
      return true;
    }
    if (first == "switch") {
      inst->op = Op::Switch;
      if (!typed_operand(c, &inst->a, &inst->src_bits)) return false;
      if (c.word() != "label") { error = "malformed switch"; return false; }
      inst->target_names[0] = c.word().substr(1);
      if (!c.eat('[')) { error = "malformed switch"; return false; }
      while (!c.eat(']')) {
        Operand value;
        if (c.done() || !typed_operand(c, &value) || !value.is_constant || c.word() != "label") { if (error.empty()) error = "malformed switch case"; return false; }
        inst->case_names.emplace_back(value.constant, c.word().substr(1));
      }
      return true;
    }
    if (first == "ret") {
      inst->op = Op::Ret;
      return true;
    }
    if (first == "call" || first == "tail" || first == "notail" || first == "musttail") {
      if (first != "call" && c.word() != "call") { error = "malformed call"; return false; }
      std::string type = c.word();
      while (type == "noundef" || type == "signext" || type == "zeroext") type = c.word();
      bool returns = false;
      if (type != "void") {
        if (!parse_int_type(type, &inst->bits)) { error = "call returning '" + type + "' is outside the integer subset"; return false; }
        returns = true;
      }
      const std::string callee = c.word();
      if (callee.empty() || callee[0] != '@') { error = "indirect calls are outside the subset"; return false; }
      if (!c.eat('(')) { error = "malformed call"; return false; }
      while (!c.eat(')')) {
        if (c.done()) { error = "unterminated call"; return false; }
        Operand value;
        int bits = 0;
        std::string arg_type = c.word();
        if (!parse_int_type(arg_type, &bits)) { error = "call argument of type '" + arg_type + "' is outside the integer subset"; return false; }
        std::string attr = c.peek_word();
        while (attr == "noundef" || attr == "signext" || attr == "zeroext") { c.word(); attr = c.peek_word(); }
        if (!operand(c, bits, &value)) return false;
        inst->args.push_back(value);
      }
      const std::string name = callee.substr(1);
      static const std::map<std::string, Op> minmax = {{"llvm.smin", Op::SMin}, {"llvm.smax", Op::SMax}, {"llvm.umin", Op::UMin}, {"llvm.umax", Op::UMax}};
      for (const auto &entry : minmax)
        if (name.compare(0, entry.first.size() + 1, entry.first + ".") == 0) {
          if (inst->args.size() != 2 || !returns) { error = "malformed min/max intrinsic"; return false; }
          inst->op = entry.second;
          inst->a = inst->args[0];
          inst->b = inst->args[1];
          return true;
        }
      inst->op = Op::Call;
      inst->command = find_command(name, &inst->operation);
      if (inst->command < 0) { error = "call to @" + name + " is outside the executed command set"; return false; }
      const CommandInfo &info = kCommands[inst->command];
      if (static_cast<int>(inst->args.size()) != info.argc || returns != info.returns_value) {
        error = "call to @" + name + " does not match its descriptor";
        return false;
      }
      return true;
    }
    error = "instruction '" + first + "' is outside the closed integer subset";
    return false;
  }

  // `!{i64 3, !"text", !7}` -> fields
  bool parse_meta_fields(const std::string &body, std::vector<MetaField> *fields) {
    size_t at = 0;
    while (at < body.size()) {
      while (at < body.size() && (body[at] == ' ' || body[at] == ',')) ++at;
      if (at >= body.size()) break;
      MetaField field;
      if (body[at] == '!' && at + 1 < body.size() && body[at + 1] == '"') {
        const size_t close = body.find('"', at + 2);
        if (close == std::string::npos) { error = "unterminated metadata string"; return false; }
        field.is_string = true;
        field.text = body.substr(at + 2, close - at - 2);
        at = close + 1;
      } else if (body[at] == '!') {
        size_t end = at + 1;
        while (end < body.size() && isdigit(static_cast<unsigned char>(body[end]))) ++end;
        field.node = atoi(body.substr(at + 1, end - at - 1).c_str());
        at = end;
      } else {
        size_t end = body.find(',', at);
        if (end == std::string::npos) end = body.size();
        const std::string item = body.substr(at, end - at);   // e.g. "i64 14"
        const size_t space = item.rfind(' ');
        field.integer = strtoll(item.c_str() + (space == std::string::npos ? 0 : space + 1), nullptr, 10);
        at = end;
      }
      fields->push_back(field);
    }
    return true;
  }

  bool parse_metadata_line(const std::string &line) {
    const size_t eq = line.find('=');
    const size_t open = line.find("!{", eq == std::string::npos ? 0 : eq);
    const size_t close = line.rfind('}');
    if (eq == std::string::npos || open == std::string::npos || close == std::string::npos || close < open) return true;  // not a tuple
    std::string name = line.substr(0, eq);
    while (!name.empty() && name.back() == ' ') name.pop_back();
    std::vector<MetaField> fields;
    if (!parse_meta_fields(line.substr(open + 2, close - open - 2), &fields)) return false;
    if (name.size() > 1 && isdigit(static_cast<unsigned char>(name[1]))) nodes[atoi(name.c_str() + 1)] = fields;
    else named[name.substr(1)] = fields;
    return true;
  }

  bool parse(const std::string &text) {
    size_t at = 0;
    bool in_function = false, saw_entry = false;
    std::string pending;   // a switch spread over several lines
    while (at <= text.size()) {
      size_t end = text.find('\n', at);
      if (end == std::string::npos) end = text.size();
      std::string line = text.substr(at, end - at);
      at = end + 1;
      if (!in_function && !line.empty() && line[0] == '!') {
        if (!parse_metadata_line(line)) return false;
        continue;
      }
      const size_t comment = line.find(';');
      if (comment != std::string::npos) line.erase(comment);
      while (!line.empty() && (line.back() == ' ' || line.back() == '\r' || line.back() == '\t')) line.pop_back();
      size_t lead = 0;
      while (lead < line.size() && (line[lead] == ' ' || line[lead] == '\t')) ++lead;
      line.erase(0, lead);
      if (line.empty()) continue;
      if (!in_function) {
        if (line.compare(0, 7, "define ") == 0) {
          if (saw_entry) { error = "a Tile module must define exactly one function"; return false; }
          saw_entry = true;
          in_function = true;
          const size_t open = line.find('('), close = line.rfind(')');
          if (open == std::string::npos || close == std::string::npos) { error = "malformed define"; return false; }
          Cursor c(line);
          c.at = open + 1;
          int unnamed = 0;
          while (c.at < close) {
            const std::string type = c.word();
            if (type.empty()) break;
            int bits = 0;
            if (!parse_int_type(type, &bits)) { error = "entry parameter of type '" + type + "' is outside the integer subset"; return false; }
            std::string name = c.peek_word();
            while (name == "noundef" || name == "signext" || name == "zeroext") { c.word(); name = c.peek_word(); }
            if (!name.empty() && name[0] == '%') { c.word(); }
            else name = "%" + std::to_string(unnamed);
            if (isdigit(static_cast<unsigned char>(name[1]))) ++unnamed;
            if (reg_of(name) != module.arg_count) { error = "duplicate entry parameter"; return false; }
            ++module.arg_count;
          }
          Block entry;
          entry.label = std::to_string(unnamed);   // the implicit number of the unnamed entry block
          module.blocks.push_back(entry);
        }
        continue;   // declarations, target triple, source_filename
      }
      if (line == "}") { in_function = false; continue; }
      if (!pending.empty()) {
        pending += " " + line;
        if (line.find(']') == std::string::npos) continue;
        line = pending;
        pending.clear();
      } else if (line.compare(0, 7, "switch ") == 0 && line.find(']') == std::string::npos) {
        pending = line;
        continue;
      }
      if (line.back() == ':') {
        Block block;
        block.label = line.substr(0, line.size() - 1);
        module.blocks.push_back(block);
        continue;
      }
      Inst inst;
      if (!parse_instruction(line, &inst)) { error += " in '" + line + "'"; return false; }
      module.blocks.back().insts.push_back(std::move(inst));
    }
    if (!saw_entry) { error = "module defines no function"; return false; }
    return resolve() && read_slots();
  }

  bool resolve() {
    std::map<std::string, int> labels;
    for (size_t b = 0; b < module.blocks.size(); ++b) labels[module.blocks[b].label] = static_cast<int>(b);
    auto find = [&](const std::string &name, int *out) {
      auto it = labels.find(name);
      if (it == labels.end()) { error = "branch to unknown block %" + name; return false; }
      *out = it->second;
      return true;
    };
    for (Block &block : module.blocks) {
      if (block.insts.empty()) { error = "block %" + block.label + " is empty"; return false; }
      const Op last = block.insts.back().op;
      if (last != Op::Br && last != Op::CondBr && last != Op::Switch && last != Op::Ret) { error = "block %" + block.label + " has no terminator"; return false; }
      block.first_non_phi = 0;
      while (block.first_non_phi < block.insts.size() && block.insts[block.first_non_phi].op == Op::Phi) ++block.first_non_phi;
      for (size_t i = 0; i < block.insts.size(); ++i) {
        Inst &inst = block.insts[i];
        if (inst.op == Op::Phi && i >= block.first_non_phi) { error = "phi after a non-phi instruction"; return false; }
        for (auto &incoming : inst.incoming_names) {
          int target;
          if (!find(incoming.second, &target)) return false;
          inst.incoming.emplace_back(incoming.first, target);
        }
        for (auto &entry : inst.case_names) {
          int target;
          if (!find(entry.second, &target)) return false;
          inst.cases.emplace_back(entry.first, target);
        }
        const int count = inst.op == Op::CondBr ? 2 : (inst.op == Op::Br || inst.op == Op::Switch) ? 1 : 0;
        for (int t = 0; t < count; ++t)
          if (!find(inst.target_names[t], &inst.targets[t])) return false;
      }
    }
    module.reg_count = static_cast<int>(regs.size());
    return true;
  }

  bool read_slots() {
    auto single = [&](const char *name, int64_t *out) {
      auto it = named.find(name);
      if (it == named.end() || it->second.size() != 1 || it->second[0].node < 0) return false;
      auto node = nodes.find(it->second[0].node);
      if (node == nodes.end() || node->second.size() != 1 || node->second[0].is_string) return false;
      *out = node->second[0].integer;
      return true;
    };
    int64_t tile = -1;
    if (!single("wafer.target.tile_id", &tile)) { error = "module carries no wafer.target.tile_id"; return false; }
    module.tile_id = static_cast<int>(tile);
    auto rows = named.find("wafer.target.entry_arguments");
    if (rows == named.end()) { error = "module carries no wafer.target.entry_arguments"; return false; }
    for (const MetaField &row : rows->second) {
      auto node = nodes.find(row.node);
      if (row.node < 0 || node == nodes.end()) { error = "dangling entry argument row"; return false; }
      const std::vector<MetaField> &f = node->second;
      // ordinal, kind, resource index, name, format, layout, byte size, alignment, access, shape..., zero-initialize
      if (f.size() < 10 || f[0].is_string || !f[1].is_string || f[2].is_string || !f[3].is_string || !f[4].is_string ||
          !f[5].is_string || f[6].is_string || f[7].is_string || !f[8].is_string) { error = "malformed entry argument row"; return false; }
      EntrySlot slot;
      slot.ordinal = f[0].integer; slot.kind = f[1].text; slot.resource = f[2].integer; slot.name = f[3].text;
      slot.format = f[4].text; slot.layout = f[5].text; slot.bytes = f[6].integer; slot.alignment = f[7].integer; slot.access = f[8].text;
      for (size_t i = 9; i + 1 < f.size(); ++i) slot.shape.push_back(f[i].integer);
      slot.zero_initialize = f.back().integer;
      if (slot.bytes <= 0 || slot.alignment <= 0) { error = "entry argument with non-positive size or alignment"; return false; }
      module.slots.push_back(slot);
    }
    if (static_cast<int>(module.slots.size()) != module.arg_count) { error = "entry arguments do not match the entry signature"; return false; }
    for (size_t i = 0; i < module.slots.size(); ++i)
      if (module.slots[i].ordinal != static_cast<int64_t>(i)) { error = "entry argument ordinals are not dense"; return false; }
    return true;
  }
};

// ------------------------------------------------------------------------------------------------ program state
constexpr uint64_t kDdrBase = 0x10000000ull;       // DDR addresses handed to the entry functions start here
constexpr uint64_t kDefaultSpmBytes = 3ull << 20;

int format_of(const std::string &name) {
  static const std::map<std::string, int> formats = {{"i8", WB200_I8}, {"i16", WB200_I16}, {"f16", WB200_F16}, {"bf16", WB200_BF16},
      {"i32", WB200_I32}, {"f32", WB200_F32}, {"tf32", WB200_TF32}, {"bool", WB200_BOOL}, {"u8", WB200_U8}, {"u16", WB200_U16},
      {"u32", WB200_U32}, {"i64", WB200_I64}, {"u64", WB200_U64}};
  auto it = formats.find(name);
  return it == formats.end() ? -1 : it->second;
}
int layout_of(const std::string &name) {
  if (name == "tensor") return WB200_LAYOUT_TENSOR;
  if (name == "ntensor") return WB200_LAYOUT_NTENSOR;
  if (name == "cx") return WB200_LAYOUT_CX;
  if (name == "ncx") return WB200_LAYOUT_NCX;
  return -1;
}

struct ExternalTensor {
  bool is_output = false;
  int64_t resource = 0;
  wb200_tensor_desc desc{};
  LayoutMap map{};
  wb200_geometry geometry{};
  uint64_t address = 0, physical_bytes = 0, compact_bytes = 0;
};

struct Endpoint {
  uint64_t event = 0;
  bool is_send = false;
  int owner = -1;
  uint64_t source = 0, destination = 0;
  uint32_t bytes = 0, local_tile = 0, remote_tile = 0, fsm = 0;
  bool peer_ready = false, matched = false, complete = false, released = false;
};
struct PreparedSend {
  uint64_t event = 0;
  int owner = -1;
  uint64_t source = 0, destination = 0;
  uint32_t bytes = 0, local_tile = 0, remote_tile = 0, fsm = 0;
  bool issued = false, released = false;
};

// Elementwise commands of one Tile that are held back while the following command may extend them into one fused launch.
struct PendingChain {
  ElementwiseChain chain{};                 // device pointers; chain.steps == 0 when nothing is pending
  uint64_t bytes = 0, lhs_address = 0;
  uint64_t rhs_address[kMaxChainSteps] = {0}, dst_address[kMaxChainSteps] = {0};
  bool rhs_vector[kMaxChainSteps] = {false};
  uint64_t first_args[8] = {0};             // the first command as issued: a chain that stays one command long runs unfused
  uint32_t first_operation = 0;
  int first_command = 0;
};

// Formal commands of one Tile (GEMMs, reductions and the elementwise commands between them) that are held back while
// the following command may join them in one launch (FormalRun): the command run of an online-attention step - scores,
// running maximum, probabilities, running sum, PV product - becomes one kernel instead of one per command.
struct PendingRun {
  FormalRun run;                  // run.count == 0 when nothing is pending
  uint64_t first_args[20] = {0};  // the first command as issued: a run that stays one command long uses the command's own kernel
  uint32_t first_operation = 0;
  int first_command = 0;
};

struct TileState {
  PendingChain chain;
  PendingRun run;
  std::vector<uint64_t> regs;
  int block = 0, previous = -1;
  size_t pc = 0;
  bool done = false;
  int dte_state = 0;            // 0 not begun, 1 active, 2 finished
  int pending_endpoint = -1;    // send endpoint created by a send_issue that has not yet seen its receiver
};

}  // namespace
}  // namespace wb200

using namespace wb200;

struct wb200_tile_program {
  wb200_backend *backend = nullptr;
  uint64_t spm_bytes = kDefaultSpmBytes;
  std::vector<Module> tiles;                      // index = Tile id
  std::vector<ExternalTensor> inputs, outputs;
  uint64_t ddr_bytes = 0;
  wb200_spm_image ddr{};
  std::vector<wb200_spm_image> spm;
  cudaEvent_t begin = nullptr, end = nullptr;
  // Device words of the numeric commands: [0] the OR of their IEEE flags, [2..3] the first refused convert element
  // (element << 8 | code, all ones when none). Zeroed before every run, read after it.
  uint32_t *numeric_words = nullptr;
  // Concurrent replay: one stream per Tile, Direct-DTE transfers as event edges, the whole invocation captured once
  // into a CUDA graph and relaunched on later runs.
  std::vector<cudaStream_t> tile_streams;
  std::vector<cudaEvent_t> edge_events;
  size_t edge_events_used = 0;
  cudaGraphExec_t graph[2] = {nullptr, nullptr};   // one captured invocation per GEMM policy
  wb200_program_stats graph_stats[2] = {};
  std::vector<uint8_t *> gemm_staging;              // per Tile: compact operands of the tensor-core GEMM path (3 x scratch-pad size)

  // per-run state
  std::vector<TileState> state;
  std::vector<Endpoint> endpoints;
  std::vector<PreparedSend> prepared;
  uint64_t next_event = 1;
  bool execute = false;
  bool fuse_chains = true;   // WB200_REPLAY_FUSE=0 in the environment issues every elementwise command as its own launch
  bool fuse_runs = false;    // WB200_REPLAY_RUNS=1 issues runs of GEMM / reduce / elementwise commands as one launch each (measured
                             // slower than one launch per command under the graph, so it is not the default)
  uint32_t gemm_policy = WB200_GEMM_FORMAL;
  wb200_program_stats stats{};
  std::vector<wb200_program_command> *trace = nullptr;
  bool activity = false;   // an endpoint was created since the scheduler last looked
};

namespace wb200 {
namespace {

wb200_status program_error(const wb200_tile_program *, int tile, const std::string &message) {
  return fail(WB200_ERR_INVALID_ARGUMENT, "tile " + std::to_string(tile) + ": " + message);
}

uint64_t value_of(const TileState &tile, const Operand &operand) { return operand.is_constant ? operand.constant : tile.regs[operand.reg]; }

// Plans the DDR arena: tensors shared by all Tiles are keyed by (kind, resource index), per-Tile arguments
// (workspace, transport status, profile record) get private ranges.
wb200_status plan_addresses(wb200_tile_program *program) {
  uint64_t at = 0;
  std::map<std::pair<std::string, int64_t>, uint64_t> shared;
  std::map<std::pair<std::string, int64_t>, EntrySlot> first_seen;
  auto place = [&](const EntrySlot &slot) {
    const uint64_t alignment = slot.alignment < 256 ? 256 : static_cast<uint64_t>(slot.alignment);
    at = (at + alignment - 1) / alignment * alignment;
    const uint64_t address = kDdrBase + at;
    at += static_cast<uint64_t>(slot.bytes);
    return address;
  };
  for (Module &module : program->tiles)
    for (EntrySlot &slot : module.slots) {
      const bool is_shared = slot.kind == "external-input" || slot.kind == "external-output" || slot.kind == "target-tensor" || slot.kind == "card-workspace";
      if (!is_shared) { slot.address = place(slot); continue; }
      const auto key = std::make_pair(slot.kind, slot.resource);
      auto it = shared.find(key);
      if (it == shared.end()) {
        slot.address = place(slot);
        shared[key] = slot.address;
        first_seen[key] = slot;
        if (slot.kind == "external-input" || slot.kind == "external-output") {
          ExternalTensor tensor;
          tensor.is_output = slot.kind == "external-output";
          tensor.resource = slot.resource;
          const int format = format_of(slot.format), layout = layout_of(slot.layout);
          if (format < 0 || layout < 0 || slot.shape.empty() || slot.shape.size() > WB200_MAX_RANK)
            return program_error(program, module.tile_id, "external tensor with unknown format, layout or rank");
          tensor.desc.format = static_cast<uint8_t>(format);
          tensor.desc.layout = static_cast<uint8_t>(layout);
          tensor.desc.rank = static_cast<uint8_t>(slot.shape.size());
          for (size_t d = 0; d < slot.shape.size(); ++d) tensor.desc.shape[d] = static_cast<uint64_t>(slot.shape[d]);
          wb200_status st = make_layout_map(tensor.desc, &tensor.map, &tensor.geometry);
          if (st != WB200_OK) return st;
          if (tensor.geometry.physical_bytes != slot.bytes)
            return program_error(program, module.tile_id, "external tensor byte size disagrees with its physical layout");
          tensor.address = slot.address;
          tensor.physical_bytes = static_cast<uint64_t>(slot.bytes);
          tensor.compact_bytes = static_cast<uint64_t>(tensor.geometry.compact_bytes);
          (tensor.is_output ? program->outputs : program->inputs).push_back(tensor);
        }
      } else {
        const EntrySlot &first = first_seen[key];
        if (first.bytes != slot.bytes || first.format != slot.format || first.layout != slot.layout || first.shape != slot.shape)
          return program_error(program, module.tile_id, "Tiles disagree on a shared entry argument");
        slot.address = it->second;
      }
    }
  auto by_resource = [](const ExternalTensor &a, const ExternalTensor &b) { return a.resource < b.resource; };
  std::sort(program->inputs.begin(), program->inputs.end(), by_resource);
  std::sort(program->outputs.begin(), program->outputs.end(), by_resource);
  program->ddr_bytes = (at + 255) / 256 * 256;
  return WB200_OK;
}

// ------------------------------------------------------------------------------------------------ command execution
void record(wb200_tile_program *program, int tile, int kind, const uint64_t *args, int argc, uint32_t operation = 0) {
  program->stats.commands += 1;
  if (!program->trace) return;
  wb200_program_command entry{};
  entry.tile = static_cast<uint32_t>(tile);
  entry.kind = static_cast<uint32_t>(kind);
  entry.argc = static_cast<uint32_t>(argc);
  entry.operation = operation;
  for (int i = 0; i < argc && i < 20; ++i) entry.args[i] = args[i];
  program->trace->push_back(entry);
}

StridedLayout layout_from(uint32_t inner, const uint64_t *strides, const uint64_t *iterations) {
  StridedLayout layout{};
  layout.inner_bytes = inner;
  for (int d = 0; d < 3; ++d) { layout.strides[d] = static_cast<uint32_t>(strides[d]); layout.iterations[d] = static_cast<uint32_t>(iterations[d]); }
  return layout;
}
StridedLayout contiguous_layout(uint32_t inner, uint64_t segments) {
  StridedLayout layout{};
  layout.inner_bytes = inner;
  layout.strides[0] = inner; layout.iterations[0] = static_cast<uint32_t>(segments);
  layout.strides[1] = layout.strides[2] = 0;
  layout.iterations[1] = layout.iterations[2] = 1;
  return layout;
}

wb200_status check_layout(const StridedLayout &layout, uint64_t byte_count) {
  for (int d = 0; d < 3; ++d)
    if (layout.iterations[d] == 0) return fail(WB200_ERR_INVALID_ARGUMENT, "movement iteration count must be positive");
  if (layout.inner_bytes == 0 || strided_segments(layout) * layout.inner_bytes != byte_count)
    return fail(WB200_ERR_INVALID_ARGUMENT, "movement byte_count differs from inner_bytes * segments");
  return WB200_OK;
}

}  // namespace

// Strided copy between two images with range checks; `stage` (a backend slot) is used when source and destination
// ranges overlap inside one image, so that the whole source is read before anything is written.
wb200_status enqueue_image_copy(wb200_spm_image *from_image, uint64_t source, const StridedLayout &from, wb200_spm_image *to_image,
                                uint64_t destination, const StridedLayout &to, bool execute, uint64_t *launches) {
  wb200_status st;
  const uint64_t from_span = strided_span(from), to_span = strided_span(to);
  if ((st = image_range(from_image, source, from_span, "movement source")) != WB200_OK) return st;
  if ((st = image_range(to_image, destination, to_span, "movement destination")) != WB200_OK) return st;
  if (!execute) return WB200_OK;
  wb200_backend *backend = to_image->backend;
  const uint8_t *src = from_image->device + (source - from_image->base);
  uint8_t *dst = to_image->device + (destination - to_image->base);
  const bool overlap = from_image == to_image && source < destination + to_span && destination < source + from_span;
  // DDR <-> scratch-pad copies run on the scratch-pad image's stream (the Tile that issued the command).
  cudaStream_t stream = (from_image->stream ? from_image : to_image)->work_stream();
  if (!overlap) {
    if ((st = launch_strided_copy(src, from, dst, to, stream)) != WB200_OK) return st;
    backend->launches += 1; *launches += 1;
    return WB200_OK;
  }
  const uint64_t payload = strided_segments(from) * from.inner_bytes;
  void *stage = to_image->staging;
  if (!stage || payload > to_image->bytes) {
    if (to_image->stream) return fail(WB200_ERR_LIMIT, "in-place gather / scatter larger than the image's staging area");
    if ((st = backend->buffer(9, payload, &stage)) != WB200_OK) return st;
  }
  const StridedLayout flat = contiguous_layout(from.inner_bytes, strided_segments(from));
  if ((st = launch_strided_copy(src, from, static_cast<uint8_t *>(stage), flat, stream)) != WB200_OK) return st;
  if ((st = launch_strided_copy(static_cast<const uint8_t *>(stage), flat, dst, to, stream)) != WB200_OK) return st;
  backend->launches += 2; *launches += 2;
  return WB200_OK;
}

// wafer_tx81_bit2fp / wafer_tx81_mask_move on one scratch-pad image (1-D Tensor vectors of `count` elements).
wb200_status enqueue_image_bit2fp(wb200_spm_image *image, uint64_t source, uint64_t destination, uint32_t count, uint32_t format, bool execute,
                                  uint64_t *launches) {
  if (!is_float_format(static_cast<int>(format))) return fail(WB200_ERR_UNSUPPORTED, "Bit2FP requires F16, BF16 or F32 output");
  if (count == 0) return fail(WB200_ERR_INVALID_ARGUMENT, "Bit2FP element count must be positive");
  wb200_status st;
  if ((st = image_range(image, source, (static_cast<uint64_t>(count) + 7) / 8, "Bit2FP source")) != WB200_OK) return st;
  if ((st = image_range(image, destination, static_cast<uint64_t>(count) * (format_bits(static_cast<int>(format)) / 8), "Bit2FP destination")) != WB200_OK) return st;
  if (!execute) return WB200_OK;
  if ((st = launch_bit2fp(image->device + (source - image->base), image->device + (destination - image->base), count, static_cast<int>(format),
                          image->work_stream())) != WB200_OK) return st;
  image->backend->launches += 1; *launches += 1;
  return WB200_OK;
}

wb200_status enqueue_image_mask_move(wb200_spm_image *image, uint64_t source, uint64_t mask, uint64_t destination, uint32_t count, uint32_t format,
                                     bool execute, int store, unsigned long long *d_refused, uint64_t *launches) {
  if (!is_float_format(static_cast<int>(format))) return fail(WB200_ERR_UNSUPPORTED, "MaskMove requires F16, BF16 or F32");
  if (count == 0) return fail(WB200_ERR_INVALID_ARGUMENT, "MaskMove element count must be positive");
  const uint64_t bytes = static_cast<uint64_t>(count) * (format_bits(static_cast<int>(format)) / 8);
  wb200_status st;
  if ((st = image_range(image, source, bytes, "MaskMove source")) != WB200_OK) return st;
  if ((st = image_range(image, mask, bytes, "MaskMove mask")) != WB200_OK) return st;
  if ((st = image_range(image, destination, bytes, "MaskMove destination")) != WB200_OK) return st;
  if (!execute) return WB200_OK;
  if ((st = launch_mask_move(image->device + (source - image->base), image->device + (mask - image->base), image->device + (destination - image->base),
                             count, static_cast<int>(format), store, d_refused, image->work_stream())) != WB200_OK) return st;
  image->backend->launches += 1; *launches += 1;
  return WB200_OK;
}

wb200_status enqueue_image_fill(wb200_spm_image *image, uint64_t destination, uint32_t value_bits, uint32_t count, uint32_t format,
                                bool execute, uint64_t *launches) {
  const int element = format_bits(static_cast<int>(format)) / 8;
  if (element != 1 && element != 2 && element != 4) return fail(WB200_ERR_UNSUPPORTED, "memset format must have 1, 2 or 4 byte elements");
  wb200_status st = image_range(image, destination, static_cast<uint64_t>(count) * element, "memset destination");
  if (st != WB200_OK || !execute) return st;
  if ((st = launch_fill(image->device + (destination - image->base), value_bits, count, element, image->work_stream())) != WB200_OK) return st;
  image->backend->launches += 1; *launches += 1;
  return WB200_OK;
}

namespace {

// An event from the program's pool (events only carry dependencies, no timing).
wb200_status program_event(wb200_tile_program *program, cudaEvent_t *event) {
  if (program->edge_events_used == program->edge_events.size()) {
    cudaEvent_t fresh;
    WB200_CUDA_CHECK(cudaEventCreateWithFlags(&fresh, cudaEventDisableTiming));
    program->edge_events.push_back(fresh);
  }
  *event = program->edge_events[program->edge_events_used++];
  return WB200_OK;
}

enum class StepResult { Progress, Blocked, Done, Failed };

// Matches endpoint `index` against the live endpoints of the opposite kind; on a match the payload is copied from
// the sender's scratch-pad to the receiver's and both sides complete.
wb200_status flush_chain(wb200_tile_program *program, int tile_index);

wb200_status try_match(wb200_tile_program *program, size_t index) {
  Endpoint &endpoint = program->endpoints[index];
  for (size_t other_index = 0; other_index < program->endpoints.size(); ++other_index) {
    if (other_index == index) continue;
    Endpoint &other = program->endpoints[other_index];
    if (other.is_send == endpoint.is_send) {
      if (!other.complete && other.local_tile == endpoint.local_tile && other.remote_tile == endpoint.remote_tile && other.fsm == endpoint.fsm)
        return program_error(program, endpoint.owner, "duplicate live Direct-DTE endpoint binding");
      continue;
    }
    if (other.matched) continue;
    Endpoint &send = endpoint.is_send ? endpoint : other;
    Endpoint &receive = endpoint.is_send ? other : endpoint;
    if (send.local_tile != receive.remote_tile || send.remote_tile != receive.local_tile || send.fsm != receive.fsm) continue;
    if (send.bytes != receive.bytes || send.destination != receive.destination)
      return program_error(program, send.owner, "matched Direct-DTE endpoints disagree on bytes or destination");
    wb200_spm_image *from = program->execute ? &program->spm[send.owner] : nullptr;
    wb200_spm_image *to = program->execute ? &program->spm[receive.owner] : nullptr;
    if (send.source + send.bytes > program->spm_bytes || receive.destination + receive.bytes > program->spm_bytes)
      return program_error(program, send.owner, "Direct-DTE transfer lies outside the scratch-pad");
    if (program->execute) {
      // Elementwise commands either Tile issued before this point may still be held back for fusion: they precede the
      // transfer in the command order (and may produce the payload or touch its destination), so they are launched first.
      wb200_status flushed;
      if ((flushed = flush_chain(program, send.owner)) != WB200_OK || (flushed = flush_chain(program, receive.owner)) != WB200_OK) return flushed;
      cudaStream_t sender = from->work_stream(), receiver = to->work_stream();
      if (sender != receiver) {
        // The payload is read after everything the sender has issued so far and lands after everything the receiver
        // has issued so far; the sender goes on only once it has been read.
        cudaEvent_t ready, copied;
        wb200_status st;
        if ((st = program_event(program, &ready)) != WB200_OK || (st = program_event(program, &copied)) != WB200_OK) return st;
        WB200_CUDA_CHECK(cudaEventRecord(ready, sender));
        WB200_CUDA_CHECK(cudaStreamWaitEvent(receiver, ready, 0));
        WB200_CUDA_CHECK(cudaMemcpyAsync(to->device + receive.destination, from->device + send.source, send.bytes, cudaMemcpyDeviceToDevice, receiver));
        WB200_CUDA_CHECK(cudaEventRecord(copied, receiver));
        WB200_CUDA_CHECK(cudaStreamWaitEvent(sender, copied, 0));
      } else {
        WB200_CUDA_CHECK(cudaMemcpyAsync(to->device + receive.destination, from->device + send.source, send.bytes, cudaMemcpyDeviceToDevice, receiver));
      }
    }
    program->stats.transfer_commands += 1;
    program->stats.bytes_moved += send.bytes;
    if (program->trace) {   // pseudo record: where in the command order the payload moved
      wb200_program_command entry{};
      entry.tile = static_cast<uint32_t>(send.owner);
      entry.kind = kCommandCount;
      entry.argc = 5;
      entry.args[0] = static_cast<uint64_t>(send.owner); entry.args[1] = static_cast<uint64_t>(receive.owner);
      entry.args[2] = send.source; entry.args[3] = receive.destination; entry.args[4] = send.bytes;
      program->trace->push_back(entry);
    }
    send.peer_ready = true;
    send.matched = receive.matched = true;
    send.complete = receive.complete = true;
    return WB200_OK;
  }
  return WB200_OK;
}

// Executes one wafer_tx81_* call of `tile`. Sets *blocked when the call has to wait for another Tile.
// One elementwise command as issued: unary (source, destination, count, format); binary (lhs, rhs | scalar bits,
// destination, count, format, rhs unit, scalar flag, numeric | rhs group); logic (lhs, rhs, destination, count, format).
wb200_status issue_elementwise(wb200_tile_program *program, wb200_spm_image *spm, int command, uint32_t operation, const uint64_t *a, bool execute) {
  const bool unary = command == kElementwiseUnary, full = command == kElementwiseBinary;
  const uint64_t rhs = unary ? 0 : a[1], destination = unary ? a[1] : a[2], count = unary ? a[2] : a[3], format = unary ? a[3] : a[4];
  const uint64_t before = execute ? program->backend->launches : 0;
  const wb200_status st = enqueue_image_elementwise(spm, operation, a[0], rhs, destination, static_cast<uint32_t>(count), static_cast<uint32_t>(format),
                                                    full ? static_cast<uint32_t>(a[5]) : 0, full ? static_cast<uint32_t>(a[6]) : 0,
                                                    full ? static_cast<uint32_t>(a[7]) : 0, program->numeric_words, execute);
  if (execute) program->stats.gpu_launches += program->backend->launches - before;
  return st;
}

wb200_status issue_run_command(wb200_tile_program *program, int tile_index, int command, uint32_t operation, const uint64_t *a, RunCommand *defer,
                               bool *deferred);

// Launches the Tile's pending command run: one kernel for two or more commands, the command's own kernel for one.
wb200_status flush_run(wb200_tile_program *program, int tile_index) {
  PendingRun &pending = program->state[tile_index].run;
  if (pending.run.count == 0) return WB200_OK;
  wb200_status st;
  const int count = pending.run.count;
  pending.run.count = 0;
  if (count == 1) return issue_run_command(program, tile_index, pending.first_command, pending.first_operation, pending.first_args, nullptr, nullptr);
  DeviceGuard guard(program->backend->device);
  pending.run.count = count;
  st = launch_formal_run(pending.run, program->numeric_words, program->spm[tile_index].work_stream());
  pending.run.count = 0;
  if (st == WB200_OK) { program->backend->launches += 1; program->stats.gpu_launches += 1; }
  return st;
}

// Launches what the Tile holds back (a command run or an elementwise chain, never both): one fused kernel for two or
// more commands, the ordinary kernel for one.
wb200_status flush_chain(wb200_tile_program *program, int tile_index) {
  if (wb200_status run_status = flush_run(program, tile_index)) return run_status;
  PendingChain &pending = program->state[tile_index].chain;
  if (pending.chain.steps == 0) return WB200_OK;
  wb200_spm_image *spm = &program->spm[tile_index];
  wb200_status st;
  if (pending.chain.steps == 1) {
    st = issue_elementwise(program, spm, pending.first_command, pending.first_operation, pending.first_args, true);
  } else {
    DeviceGuard guard(program->backend->device);
    st = launch_elementwise_chain(pending.chain, program->numeric_words, spm->work_stream());
    if (st == WB200_OK) { program->backend->launches += 1; program->stats.gpu_launches += 1; }
  }
  pending.chain.steps = 0;
  return st;
}

// Two equally long byte ranges may both take part in a chain when they coincide or do not touch: a thread of the fused
// kernel owns the same elements of every vector, so only a shifted overlap would cross threads.
bool ranges_compatible(uint64_t x, uint64_t y, uint64_t bytes) { return x == y || x + bytes <= y || y + bytes <= x; }

// Holds an arithmetic / function elementwise command back as a chain step, extending the pending chain when the
// command's first operand is the pending chain's last destination. Validation has already passed.
wb200_status defer_elementwise(wb200_tile_program *program, int tile_index, int command, uint32_t operation, const uint64_t *a) {
  PendingChain &pending = program->state[tile_index].chain;
  wb200_spm_image *spm = &program->spm[tile_index];
  const bool unary = command == kElementwiseUnary;
  const bool rhs_vector = !unary && a[6] == 0;
  const uint64_t lhs = a[0], rhs = unary ? 0 : a[1], destination = unary ? a[1] : a[2], count = unary ? a[2] : a[3], format = unary ? a[3] : a[4];
  const uint64_t bytes = count * (format_bits(static_cast<int>(format)) / 8);
  wb200_status st;
  bool extend = pending.chain.steps > 0 && pending.chain.steps < kMaxChainSteps && pending.chain.format == static_cast<int32_t>(format) &&
                pending.chain.count == static_cast<int64_t>(count) && lhs == pending.dst_address[pending.chain.steps - 1];
  if (extend) {
    extend = ranges_compatible(destination, pending.lhs_address, bytes) && (!rhs_vector || ranges_compatible(destination, rhs, bytes));
    for (int s = 0; extend && s < pending.chain.steps; ++s)
      extend = ranges_compatible(destination, pending.dst_address[s], bytes) &&
               (!pending.rhs_vector[s] || ranges_compatible(destination, pending.rhs_address[s], bytes)) &&
               (!rhs_vector || ranges_compatible(rhs, pending.dst_address[s], bytes));
  }
  if (!extend) {
    if ((st = flush_chain(program, tile_index)) != WB200_OK) return st;
    if (!ranges_compatible(destination, lhs, bytes) || (rhs_vector && !ranges_compatible(destination, rhs, bytes)))
      return issue_elementwise(program, spm, command, operation, a, true);   // shifted in-place command: never part of a chain
    pending.chain.format = static_cast<int32_t>(format);
    pending.chain.count = static_cast<int64_t>(count);
    pending.chain.lhs = spm->device + (lhs - spm->base);
    pending.bytes = bytes;
    pending.lhs_address = lhs;
    pending.first_command = command;
    pending.first_operation = operation;
    for (int i = 0; i < 8; ++i) pending.first_args[i] = a[i];
  }
  const int s = pending.chain.steps++;
  ChainStep &step = pending.chain.step[s];
  step.op = static_cast<int32_t>(operation);
  step.rhs_mode = rhs_vector ? WB200_RHS_SAME : WB200_RHS_SCALAR;
  step.scalar = unary ? 0u : static_cast<uint32_t>(rhs);
  step.reserved = 0;
  step.rhs = rhs_vector ? spm->device + (rhs - spm->base) : nullptr;
  step.dst = spm->device + (destination - spm->base);
  pending.rhs_vector[s] = rhs_vector;
  pending.rhs_address[s] = rhs_vector ? rhs : 0;
  pending.dst_address[s] = destination;
  return WB200_OK;
}

// One GEMM, reduction or elementwise command as issued. With `defer` nothing is launched: the command is validated and
// described, and *deferred says whether it fits a command run. Without it the command's own kernel is launched.
wb200_status issue_run_command(wb200_tile_program *program, int tile_index, int command, uint32_t operation, const uint64_t *a, RunCommand *defer,
                               bool *deferred) {
  wb200_spm_image *spm = program->execute ? &program->spm[tile_index] : nullptr;
  wb200_spm_image probe_spm{nullptr, 0, program->spm_bytes, nullptr};
  if (!program->execute) spm = &probe_spm;
  const uint64_t before = program->execute ? program->backend->launches : 0;
  wb200_status st;
  if (command == kReduce) {
    const uint32_t nhwc[4] = {static_cast<uint32_t>(a[3]), static_cast<uint32_t>(a[4]), static_cast<uint32_t>(a[5]), static_cast<uint32_t>(a[6])};
    st = enqueue_image_reduce(spm, operation, a[0], a[1], static_cast<uint32_t>(a[2]), nhwc, static_cast<uint32_t>(a[7]), program->numeric_words,
                              program->execute, defer, deferred);
  } else if (command == kGemm || command == kGemmOriented) {
    const uint32_t lhs_orientation = command == kGemmOriented ? static_cast<uint32_t>(a[11]) : WB200_NORMAL;
    const uint32_t rhs_orientation = command == kGemmOriented ? static_cast<uint32_t>(a[12]) : WB200_NORMAL;
    st = enqueue_image_gemm(spm, a[0], a[1], a[2], a[3], static_cast<uint32_t>(a[4]), static_cast<uint32_t>(a[5]), static_cast<uint32_t>(a[6]),
                            static_cast<uint32_t>(a[7]), static_cast<uint32_t>(a[8]), static_cast<uint32_t>(a[9]), static_cast<uint32_t>(a[10]),
                            lhs_orientation, rhs_orientation, program->gemm_policy, defer, deferred);
  } else {
    const bool unary = command == kElementwiseUnary, full = command == kElementwiseBinary;
    const uint64_t rhs = unary ? 0 : a[1], destination = unary ? a[1] : a[2], count = unary ? a[2] : a[3], format = unary ? a[3] : a[4];
    st = enqueue_image_elementwise(spm, operation, a[0], rhs, destination, static_cast<uint32_t>(count), static_cast<uint32_t>(format),
                                   full ? static_cast<uint32_t>(a[5]) : 0, full ? static_cast<uint32_t>(a[6]) : 0, full ? static_cast<uint32_t>(a[7]) : 0,
                                   program->numeric_words, program->execute, defer, deferred);
  }
  if (program->execute) program->stats.gpu_launches += program->backend->launches - before;
  return st;
}

// Tries to add the command to the Tile's pending run. *joined is false when the command does not fit a run (too large,
// tensor-core GEMM policy): the pending run has then been launched and the caller issues the command on its own.
wb200_status join_run(wb200_tile_program *program, int tile_index, int command, uint32_t operation, const uint64_t *a, bool *joined) {
  PendingRun &pending = program->state[tile_index].run;
  *joined = false;
  RunCommand described;
  bool fits = false;
  wb200_status st = issue_run_command(program, tile_index, command, operation, a, &described, &fits);
  if (st != WB200_OK) return st;
  if (!fits) return flush_chain(program, tile_index);
  if (pending.run.count == kMaxRunCommands && (st = flush_run(program, tile_index)) != WB200_OK) return st;
  if (pending.run.count == 0) {
    pending.first_command = command;
    pending.first_operation = operation;
    for (int i = 0; i < 20; ++i) pending.first_args[i] = a[i];
  }
  pending.run.command[pending.run.count++] = described;
  *joined = true;
  return WB200_OK;
}

wb200_status execute_call(wb200_tile_program *program, int tile_index, const Inst &inst, bool *blocked, uint64_t *result) {
  TileState &tile = program->state[tile_index];
  uint64_t a[20] = {0};
  const CommandInfo &info = kCommands[inst.command];
  const int argc = info.has_worker ? info.argc - 1 : info.argc;   // the trailing NCC worker does not reach the payload
  for (int i = 0; i < argc; ++i) a[i] = value_of(tile, inst.args[i]);
  if (info.has_worker && value_of(tile, inst.args[argc]) >= 4) return program_error(program, tile_index, "NCC worker outside the worker domain");
  wb200_spm_image *spm = program->execute ? &program->spm[tile_index] : nullptr;
  wb200_spm_image probe_spm{nullptr, 0, program->spm_bytes, nullptr}, probe_ddr{nullptr, kDdrBase, program->ddr_bytes, nullptr};
  if (!program->execute) spm = &probe_spm;
  wb200_spm_image *ddr = program->execute ? &program->ddr : &probe_ddr;
  wb200_status st = WB200_OK;
  *blocked = false;
  *result = 0;
  const bool elementwise = inst.command == kElementwiseUnary || inst.command == kElementwiseBinary || inst.command == kElementwiseLogic;
  const bool run_starter = inst.command == kGemm || inst.command == kGemmOriented || inst.command == kReduce;
  const bool runs = program->execute && program->fuse_chains && program->fuse_runs;
  // Held-back commands precede this one, unless it may join them: a GEMM or a reduction joins (or opens) a command run,
  // an elementwise command joins an open run or the elementwise chain.
  if (!elementwise && !(run_starter && runs && tile.run.run.count > 0) && (st = flush_chain(program, tile_index)) != WB200_OK) return st;
  switch (inst.command) {
    case kNccJoin:
      if (a[0] == 0 || (a[0] & ~0xFull)) return program_error(program, tile_index, "NCC join mask is empty or outside the worker domain");
      record(program, tile_index, inst.command, a, argc);
      program->stats.sync_commands += 1;   // commands of one Tile already run in issue order on the stream
      return WB200_OK;
    case kDteBegin:
    case kDteBeginAfterPrepare:
      if (tile.dte_state != 0) return program_error(program, tile_index, "Direct-DTE begin is duplicate or follows finish");
      if (a[1] != program->tiles.size()) return program_error(program, tile_index, "Direct-DTE participant count differs from the Tile count");
      tile.dte_state = 1;
      record(program, tile_index, inst.command, a, argc);
      program->stats.sync_commands += 1;
      return WB200_OK;
    case kDteFinish:
      if (tile.dte_state != 1) return program_error(program, tile_index, "Direct-DTE finish without begin");
      for (const Endpoint &endpoint : program->endpoints)
        if (endpoint.owner == tile_index && !endpoint.released) return program_error(program, tile_index, "Direct-DTE finish with a live endpoint");
      tile.dte_state = 2;
      record(program, tile_index, inst.command, a, argc);
      program->stats.sync_commands += 1;
      return WB200_OK;
    case kDteSendPrepare: {
      if (tile.dte_state != 1) return program_error(program, tile_index, "Direct-DTE send prepare outside begin / finish");
      if (a[3] != static_cast<uint64_t>(tile_index)) return program_error(program, tile_index, "Direct-DTE send names a foreign local Tile");
      if (a[4] >= program->tiles.size() || a[6] > 1) return program_error(program, tile_index, "Direct-DTE send names an unknown Tile or flag");
      for (const PreparedSend &send : program->prepared)
        if (send.owner == tile_index && !send.released) return program_error(program, tile_index, "sender already has a live prepared event");
      PreparedSend send;
      send.event = program->next_event++;
      send.owner = tile_index;
      send.source = a[0]; send.destination = a[1]; send.bytes = static_cast<uint32_t>(a[2]);
      send.local_tile = static_cast<uint32_t>(a[3]); send.remote_tile = static_cast<uint32_t>(a[4]); send.fsm = static_cast<uint32_t>(a[5]);
      program->prepared.push_back(send);
      record(program, tile_index, inst.command, a, argc);
      *result = send.event;
      return WB200_OK;
    }
    case kDteSendIssue: {
      if (tile.pending_endpoint < 0) {
        if (tile.dte_state != 1) return program_error(program, tile_index, "Direct-DTE send issue outside begin / finish");
        PreparedSend *prepared = nullptr;
        for (PreparedSend &send : program->prepared)
          if (send.event == a[0]) prepared = &send;
        if (!prepared || prepared->owner != tile_index || prepared->issued || prepared->released)
          return program_error(program, tile_index, "send issue names an unknown, foreign or already issued event");
        Endpoint endpoint;
        endpoint.event = prepared->event; endpoint.is_send = true; endpoint.owner = tile_index;
        endpoint.source = prepared->source; endpoint.destination = prepared->destination; endpoint.bytes = prepared->bytes;
        endpoint.local_tile = prepared->local_tile; endpoint.remote_tile = prepared->remote_tile; endpoint.fsm = prepared->fsm;
        prepared->issued = true;
        program->endpoints.push_back(endpoint);
        tile.pending_endpoint = static_cast<int>(program->endpoints.size() - 1);
        program->activity = true;
        record(program, tile_index, inst.command, a, argc);
        if ((st = try_match(program, program->endpoints.size() - 1)) != WB200_OK) return st;
      }
      if (!program->endpoints[tile.pending_endpoint].peer_ready) { *blocked = true; return WB200_OK; }   // returns once the receiver is prepared
      tile.pending_endpoint = -1;
      return WB200_OK;
    }
    case kDteRecvPrepare: {
      if (tile.dte_state != 1) return program_error(program, tile_index, "Direct-DTE receive outside begin / finish");
      if (a[2] != static_cast<uint64_t>(tile_index)) return program_error(program, tile_index, "Direct-DTE receive names a foreign local Tile");
      if (a[3] >= program->tiles.size()) return program_error(program, tile_index, "Direct-DTE receive names an unknown Tile");
      Endpoint endpoint;
      endpoint.event = program->next_event++; endpoint.is_send = false; endpoint.owner = tile_index;
      endpoint.destination = a[0]; endpoint.bytes = static_cast<uint32_t>(a[1]);
      endpoint.local_tile = static_cast<uint32_t>(a[2]); endpoint.remote_tile = static_cast<uint32_t>(a[3]); endpoint.fsm = static_cast<uint32_t>(a[4]);
      endpoint.peer_ready = true;
      program->endpoints.push_back(endpoint);
      record(program, tile_index, inst.command, a, argc);
      *result = endpoint.event;
      return try_match(program, program->endpoints.size() - 1);
    }
    case kDteWait: {
      bool any = false, all_complete = true;
      for (PreparedSend &send : program->prepared)
        if (send.event == a[0] && send.owner == tile_index && !send.issued)
          return program_error(program, tile_index, "wait names a prepared send that was not issued");
      for (Endpoint &endpoint : program->endpoints)
        if (endpoint.event == a[0] && endpoint.owner == tile_index) {
          if (endpoint.released) return program_error(program, tile_index, "wait names an already released event");
          any = true;
          all_complete = all_complete && endpoint.complete;
        }
      if (!any) return program_error(program, tile_index, "wait names an unknown or foreign event");
      if (!all_complete) { *blocked = true; return WB200_OK; }
      for (Endpoint &endpoint : program->endpoints)
        if (endpoint.event == a[0] && endpoint.owner == tile_index) endpoint.released = true;
      for (PreparedSend &send : program->prepared)
        if (send.event == a[0] && send.owner == tile_index) send.released = true;
      record(program, tile_index, inst.command, a, argc);
      program->stats.sync_commands += 1;
      return WB200_OK;
    }
    case kRdma:
    case kWdma: {
      // (source, destination, byte_count, inner_bytes, strides[3], iterations[3], format)
      const StridedLayout strided = layout_from(static_cast<uint32_t>(a[3]), a + 4, a + 7);
      if ((st = check_layout(strided, a[2])) != WB200_OK) return st;
      const StridedLayout flat = contiguous_layout(strided.inner_bytes, strided_segments(strided));
      record(program, tile_index, inst.command, a, argc);
      program->stats.movement_commands += 1;
      program->stats.bytes_moved += a[2];
      if (inst.command == kRdma) return enqueue_image_copy(ddr, a[0], strided, spm, a[1], flat, program->execute, &program->stats.gpu_launches);
      return enqueue_image_copy(spm, a[0], flat, ddr, a[1], strided, program->execute, &program->stats.gpu_launches);
    }
    case kGatherScatter: {
      // (source, destination, byte_count, inner_bytes, src strides[3], src iterations[3], dst strides[3], dst iterations[3])
      const StridedLayout from = layout_from(static_cast<uint32_t>(a[3]), a + 4, a + 7);
      const StridedLayout to = layout_from(static_cast<uint32_t>(a[3]), a + 10, a + 13);
      if ((st = check_layout(from, a[2])) != WB200_OK || (st = check_layout(to, a[2])) != WB200_OK) return st;
      record(program, tile_index, inst.command, a, argc);
      program->stats.movement_commands += 1;
      program->stats.bytes_moved += a[2];
      return enqueue_image_copy(spm, a[0], from, spm, a[1], to, program->execute, &program->stats.gpu_launches);
    }
    case kMemset:
      // (destination, value, element_count, format)
      record(program, tile_index, inst.command, a, argc);
      program->stats.fill_commands += 1;
      program->stats.bytes_moved += a[2] * (format_bits(static_cast<int>(a[3])) / 8);
      return enqueue_image_fill(spm, a[0], static_cast<uint32_t>(a[1]), static_cast<uint32_t>(a[2]), static_cast<uint32_t>(a[3]), program->execute,
                                &program->stats.gpu_launches);
    case kElementwiseUnary:
    case kElementwiseBinary:
    case kElementwiseLogic: {
      const bool unary = inst.command == kElementwiseUnary, full = inst.command == kElementwiseBinary;
      const uint64_t count = unary ? a[2] : a[3], format = unary ? a[3] : a[4];
      record(program, tile_index, inst.command, a, argc, inst.operation);
      program->stats.bytes_moved += count * (format_bits(static_cast<int>(format)) / 8) * (unary ? 2 : 3);
      if (!program->execute || !program->fuse_chains) return issue_elementwise(program, spm, inst.command, inst.operation, a, program->execute);
      if ((st = issue_elementwise(program, spm, inst.command, inst.operation, a, false)) != WB200_OK) return st;   // validation only
      if (tile.run.run.count > 0) {
        bool joined = false;
        if ((st = join_run(program, tile_index, inst.command, inst.operation, a, &joined)) != WB200_OK || joined) return st;
      }
      const uint32_t op = inst.operation;
      const bool arithmetic = op == WB200_EW_MAX || op == WB200_EW_MIN || op == WB200_EW_ADD || op == WB200_EW_SUB || op == WB200_EW_MUL;
      // same-index or immediate second operands only; relations, logic and the repeated-unit / grouped forms run unfused
      const bool chainable = unary ? op != WB200_EW_LOGIC_NOT : (full && arithmetic && (a[6] != 0 || (a[5] == 0 && a[7] == 0)));
      if (chainable) return defer_elementwise(program, tile_index, inst.command, op, a);
      if ((st = flush_chain(program, tile_index)) != WB200_OK) return st;
      return issue_elementwise(program, spm, inst.command, op, a, true);
    }
    case kPool: {
      // (input, destination, kind, source nhwc[4], destination nhwc[4], pads[4], kernel w / h and stride w / h, format)
      if (a[2] != inst.operation) return program_error(program, tile_index, "pool kind field differs from the symbol's operation");
      uint32_t fields[16];
      for (int i = 0; i < 16; ++i) fields[i] = static_cast<uint32_t>(a[3 + i]);
      record(program, tile_index, inst.command, a, argc, inst.operation);
      const uint64_t before = program->execute ? program->backend->launches : 0;
      st = enqueue_image_pool(spm, inst.operation, a[0], a[1], fields, fields + 4, fields + 8, fields + 12, static_cast<uint32_t>(a[19]),
                              program->numeric_words, program->execute);
      if (program->execute) program->stats.gpu_launches += program->backend->launches - before;
      return st;
    }
    case kBit2Fp:
      // (source, destination, count, format)
      record(program, tile_index, inst.command, a, argc);
      program->stats.bytes_moved += (a[2] + 7) / 8 + a[2] * (format_bits(static_cast<int>(a[3])) / 8);
      return enqueue_image_bit2fp(spm, a[0], a[1], static_cast<uint32_t>(a[2]), static_cast<uint32_t>(a[3]), program->execute, &program->stats.gpu_launches);
    case kMaskMove:
      // (source, mask, destination, count, format); a mask value other than 0 / 1.0 fails the run after the stream drains
      record(program, tile_index, inst.command, a, argc);
      program->stats.bytes_moved += 3 * a[3] * (format_bits(static_cast<int>(a[4])) / 8);
      return enqueue_image_mask_move(spm, a[0], a[1], a[2], static_cast<uint32_t>(a[3]), static_cast<uint32_t>(a[4]), program->execute, 1,
                                     reinterpret_cast<unsigned long long *>(program->numeric_words + 2), &program->stats.gpu_launches);
    case kReduce: {
      // (source, destination, dimension, n, h, w, c, format)
      record(program, tile_index, inst.command, a, argc, inst.operation);
      if (runs) {
        bool joined = false;
        if ((st = join_run(program, tile_index, inst.command, inst.operation, a, &joined)) != WB200_OK || joined) return st;
      }
      return issue_run_command(program, tile_index, inst.command, inst.operation, a, nullptr, nullptr);
    }
    case kConvert: {
      // (source, destination, count, zero point, rounding mode)
      record(program, tile_index, inst.command, a, argc, inst.operation);
      const uint64_t before = program->execute ? program->backend->launches : 0;
      st = enqueue_image_convert(spm, inst.operation, a[0], a[1], static_cast<uint32_t>(a[2]), static_cast<uint32_t>(a[4]), program->execute,
                                 program->numeric_words, reinterpret_cast<unsigned long long *>(program->numeric_words + 2));
      if (program->execute) program->stats.gpu_launches += program->backend->launches - before;
      return st;
    }
    case kGemm:
    case kGemmOriented: {
      // (lhs, rhs, dst, psum, m, k, n, batch, in format, out format, psum format[, lhs orientation, rhs orientation])
      const uint32_t lhs_orientation = inst.command == kGemmOriented ? static_cast<uint32_t>(a[11]) : WB200_NORMAL;
      const uint32_t rhs_orientation = inst.command == kGemmOriented ? static_cast<uint32_t>(a[12]) : WB200_NORMAL;
      if (lhs_orientation > 1 || rhs_orientation > 1) return program_error(program, tile_index, "unknown GEMM orientation");
      record(program, tile_index, inst.command, a, argc);
      program->stats.gemm_commands += 1;
      program->stats.gemm_fused_multiply_adds += a[4] * a[5] * a[6] * a[7];
      if (!program->execute) return WB200_OK;
      if (runs) {
        bool joined = false;
        if ((st = join_run(program, tile_index, inst.command, inst.operation, a, &joined)) != WB200_OK || joined) return st;
      }
      return issue_run_command(program, tile_index, inst.command, inst.operation, a, nullptr, nullptr);
    }
    default:
      return program_error(program, tile_index, "command outside the executed set");
  }
}

uint64_t evaluate(const Inst &inst, uint64_t a, uint64_t b, uint64_t c, bool *division_by_zero) {
  const int bits = inst.bits;
  switch (inst.op) {
    case Op::Add: return mask_to(a + b, bits);
    case Op::Sub: return mask_to(a - b, bits);
    case Op::Mul: return mask_to(a * b, bits);
    case Op::UDiv: if (b == 0) { *division_by_zero = true; return 0; } return a / b;
    case Op::URem: if (b == 0) { *division_by_zero = true; return 0; } return a % b;
    case Op::SDiv:
    case Op::SRem: {
      const int64_t x = sign_extend(a, bits), y = sign_extend(b, bits);
      if (y == 0 || (y == -1 && x == sign_extend(uint64_t(1) << (bits - 1), bits))) { *division_by_zero = true; return 0; }
      return mask_to(static_cast<uint64_t>(inst.op == Op::SDiv ? x / y : x % y), bits);
    }
    case Op::And: return a & b;
    case Op::Or: return a | b;
    case Op::Xor: return a ^ b;
    case Op::Shl: return b >= static_cast<uint64_t>(bits) ? 0 : mask_to(a << b, bits);
    case Op::LShr: return b >= static_cast<uint64_t>(bits) ? 0 : a >> b;
    case Op::AShr: return mask_to(static_cast<uint64_t>(sign_extend(a, bits) >> (b >= static_cast<uint64_t>(bits) ? bits - 1 : b)), bits);
    case Op::ICmp: {
      const int64_t x = sign_extend(a, inst.src_bits), y = sign_extend(b, inst.src_bits);
      switch (inst.pred) {
        case Pred::Eq: return a == b; case Pred::Ne: return a != b;
        case Pred::Ugt: return a > b; case Pred::Uge: return a >= b; case Pred::Ult: return a < b; case Pred::Ule: return a <= b;
        case Pred::Sgt: return x > y; case Pred::Sge: return x >= y; case Pred::Slt: return x < y; case Pred::Sle: return x <= y;
      }
      return 0;
    }
    case Op::Select: return a ? b : c;
    case Op::ZExt: return a;
    case Op::SExt: return mask_to(static_cast<uint64_t>(sign_extend(a, inst.src_bits)), bits);
    case Op::Trunc: return mask_to(a, bits);
    case Op::Freeze: return a;
    case Op::SMin: return sign_extend(a, bits) < sign_extend(b, bits) ? a : b;
    case Op::SMax: return sign_extend(a, bits) > sign_extend(b, bits) ? a : b;
    case Op::UMin: return a < b ? a : b;
    case Op::UMax: return a > b ? a : b;
    default: return 0;
  }
}

void enter_block(const Module &module, TileState &tile, int target) {
  const Block &block = module.blocks[target];
  // phis read their incoming values simultaneously
  uint64_t staged[64];
  std::vector<uint64_t> overflow;
  const size_t count = block.first_non_phi;
  uint64_t *values = staged;
  if (count > 64) { overflow.resize(count); values = overflow.data(); }
  for (size_t i = 0; i < count; ++i) {
    const Inst &phi = block.insts[i];
    values[i] = 0;
    for (const auto &incoming : phi.incoming)
      if (incoming.second == tile.block) { values[i] = value_of(tile, incoming.first); break; }
  }
  for (size_t i = 0; i < count; ++i) tile.regs[block.insts[i].dst] = values[i];
  tile.previous = tile.block;
  tile.block = target;
  tile.pc = count;
}

// Runs `tile` until it finishes or has to wait for another Tile.
wb200_status run_tile(wb200_tile_program *program, int tile_index, StepResult *result, bool *progressed) {
  const Module &module = program->tiles[tile_index];
  TileState &tile = program->state[tile_index];
  constexpr uint64_t kInstructionLimit = 1ull << 32;
  while (true) {
    const Inst &inst = module.blocks[tile.block].insts[tile.pc];
    if (program->stats.instructions++ > kInstructionLimit) return program_error(program, tile_index, "instruction limit exceeded");
    switch (inst.op) {
      case Op::Br: enter_block(module, tile, inst.targets[0]); *progressed = true; break;
      case Op::CondBr: enter_block(module, tile, value_of(tile, inst.a) ? inst.targets[0] : inst.targets[1]); *progressed = true; break;
      case Op::Switch: {
        const uint64_t value = value_of(tile, inst.a);
        int target = inst.targets[0];
        for (const auto &entry : inst.cases)
          if (entry.first == value) { target = entry.second; break; }
        enter_block(module, tile, target);
        *progressed = true;
        break;
      }
      case Op::Ret:
        if (tile.dte_state == 1) return program_error(program, tile_index, "entry returned inside a Direct-DTE session");
        if (wb200_status st = flush_chain(program, tile_index)) return st;
        tile.done = true;
        *result = StepResult::Done;
        *progressed = true;
        return WB200_OK;
      case Op::Call: {
        bool blocked = false;
        uint64_t value = 0;
        wb200_status st = execute_call(program, tile_index, inst, &blocked, &value);
        if (st != WB200_OK) return st;
        if (blocked) { *result = StepResult::Blocked; return WB200_OK; }
        if (inst.dst >= 0) tile.regs[inst.dst] = value;
        tile.pc += 1;
        *progressed = true;
        break;
      }
      case Op::Phi:
        return program_error(program, tile_index, "phi reached outside block entry");
      default: {
        bool division_by_zero = false;
        const uint64_t value = evaluate(inst, value_of(tile, inst.a), value_of(tile, inst.b), value_of(tile, inst.c), &division_by_zero);
        if (division_by_zero) return program_error(program, tile_index, "integer division by zero or overflow");
        tile.regs[inst.dst] = value;
        tile.pc += 1;
        *progressed = true;
        break;
      }
    }
  }
}

// Cooperative scheduling: every Tile runs until it blocks; a full round without progress is a deadlock.
wb200_status run_all_tiles(wb200_tile_program *program) {
  const size_t count = program->tiles.size();
  program->state.assign(count, TileState{});
  program->endpoints.clear();
  program->prepared.clear();
  program->next_event = 1;
  program->stats = wb200_program_stats{};
  for (size_t t = 0; t < count; ++t) {
    TileState &tile = program->state[t];
    tile.regs.assign(program->tiles[t].reg_count, 0);
    for (int a = 0; a < program->tiles[t].arg_count; ++a) tile.regs[a] = program->tiles[t].slots[a].address;
    tile.pc = program->tiles[t].blocks[0].first_non_phi;
  }
  size_t remaining = count;
  while (remaining > 0) {
    bool progressed = false;
    program->activity = false;
    for (size_t t = 0; t < count; ++t) {
      if (program->state[t].done) continue;
      StepResult result = StepResult::Progress;
      wb200_status st = run_tile(program, static_cast<int>(t), &result, &progressed);
      if (st != WB200_OK) return st;
      if (result == StepResult::Done) --remaining;
    }
    if (!progressed && !program->activity && remaining > 0) {
      std::string waiting;
      for (size_t t = 0; t < count; ++t)
        if (!program->state[t].done) waiting += (waiting.empty() ? "" : ", ") + std::to_string(t);
      return fail(WB200_ERR_INVALID_ARGUMENT, "Tiles " + waiting + " wait on Direct-DTE endpoints that nothing completes (deadlock)");
    }
  }
  for (const Endpoint &endpoint : program->endpoints)
    if (!endpoint.matched) return program_error(program, endpoint.owner, "invocation ended with an unmatched Direct-DTE endpoint");
  return WB200_OK;
}

}  // namespace
}  // namespace wb200

namespace wb200 {
namespace {

// Interprets the invocation once while the backend stream and the Tile streams are being captured: every Tile's
// commands land on its own stream, Direct-DTE transfers become event edges between streams, and the result is one
// instantiated CUDA graph whose branches run concurrently on later launches.
wb200_status capture_invocation(wb200_tile_program *program) {
  wb200_backend *backend = program->backend;
  cudaStream_t origin = backend->stream;
  const uint32_t policy = program->gemm_policy;
  if (policy == WB200_GEMM_TENSOR) {
    // Nothing may allocate or set launch attributes while the streams are being captured: the Tiles' private areas for
    // the compact GEMM operands (the backend's slots would be shared by Tiles that now run side by side) and the
    // kernels' attributes come first.
    if (program->gemm_staging.empty()) {
      program->gemm_staging.assign(program->spm.size(), nullptr);
      for (size_t t = 0; t < program->spm.size(); ++t) WB200_CUDA_CHECK(cudaMalloc(&program->gemm_staging[t], 3 * program->spm_bytes));
    }
    wb200_status prepared = gemm_umma_prepare();
    if (prepared != WB200_OK) return prepared;
  }
  for (size_t t = 0; t < program->spm.size(); ++t) {
    program->spm[t].stream = program->tile_streams[t];
    program->spm[t].staging = program->spm[t].device + program->spm_bytes;
    program->spm[t].gemm_staging = policy == WB200_GEMM_TENSOR ? program->gemm_staging[t] : nullptr;
  }
  program->edge_events_used = 0;
  cudaEvent_t fork;
  wb200_status st = program_event(program, &fork);
  if (st != WB200_OK) return st;
  WB200_CUDA_CHECK(cudaStreamBeginCapture(origin, cudaStreamCaptureModeThreadLocal));
  cudaError_t err = cudaEventRecord(fork, origin);
  for (size_t t = 0; err == cudaSuccess && t < program->tile_streams.size(); ++t) err = cudaStreamWaitEvent(program->tile_streams[t], fork, 0);
  if (err == cudaSuccess) {
    st = run_all_tiles(program);
    for (size_t t = 0; st == WB200_OK && t < program->tile_streams.size(); ++t) {
      cudaEvent_t joined;
      if ((st = program_event(program, &joined)) != WB200_OK) break;
      if ((err = cudaEventRecord(joined, program->tile_streams[t])) != cudaSuccess) break;
      if ((err = cudaStreamWaitEvent(origin, joined, 0)) != cudaSuccess) break;
    }
  }
  cudaGraph_t graph = nullptr;
  const cudaError_t end_error = cudaStreamEndCapture(origin, &graph);   // always leave capture mode
  if (st == WB200_OK && err != cudaSuccess) st = fail(WB200_ERR_CUDA, std::string("capturing the invocation: ") + cudaGetErrorString(err));
  if (st == WB200_OK && end_error != cudaSuccess) st = fail(WB200_ERR_CUDA, std::string("ending the capture: ") + cudaGetErrorString(end_error));
  if (st != WB200_OK) {
    if (graph) cudaGraphDestroy(graph);
    cudaGetLastError();
    return st;
  }
  err = cudaGraphInstantiate(&program->graph[policy], graph, 0);
  cudaGraphDestroy(graph);
  if (err != cudaSuccess) { program->graph[policy] = nullptr; return fail(WB200_ERR_CUDA, std::string("instantiating the invocation graph: ") + cudaGetErrorString(err)); }
  program->graph_stats[policy] = program->stats;
  return WB200_OK;
}

}  // namespace
}  // namespace wb200

extern "C" {

const char *wb200_program_command_name(uint32_t kind) {
  if (kind == kCommandCount) return "direct_dte_transfer";   // trace-only record: (sender Tile, receiver Tile, source, destination, bytes)
  return kind < kCommandCount ? kCommands[kind].symbol : "";
}

wb200_status wb200_tile_program_load(wb200_backend *backend, const char *const *module_texts, uint32_t tile_count, uint64_t spm_bytes,
                                     wb200_tile_program **out) {
  if (!module_texts || !out || tile_count == 0 || tile_count > 1024) return fail(WB200_ERR_INVALID_ARGUMENT, "invalid Tile program request");
  std::unique_ptr<wb200_tile_program> program(new wb200_tile_program);
  program->backend = backend;
  program->spm_bytes = spm_bytes ? spm_bytes : kDefaultSpmBytes;
  { const char *env = getenv("WB200_REPLAY_FUSE"); program->fuse_chains = !(env && env[0] == '0'); }
  { const char *env = getenv("WB200_REPLAY_RUNS"); program->fuse_runs = env && env[0] == '1'; }
  program->tiles.resize(tile_count);
  std::vector<bool> seen(tile_count, false);
  for (uint32_t i = 0; i < tile_count; ++i) {
    if (!module_texts[i]) return fail(WB200_ERR_INVALID_ARGUMENT, "null module text");
    ModuleParser parser;
    if (!parser.parse(module_texts[i])) {
      const bool unsupported = parser.error.find("outside") != std::string::npos;
      return fail(unsupported ? WB200_ERR_UNSUPPORTED : WB200_ERR_INVALID_ARGUMENT, "module " + std::to_string(i) + ": " + parser.error);
    }
    const int tile = parser.module.tile_id;
    if (tile < 0 || tile >= static_cast<int>(tile_count) || seen[tile]) return fail(WB200_ERR_INVALID_ARGUMENT, "Tile ids are not a permutation of 0..count-1");
    seen[tile] = true;
    program->tiles[tile] = std::move(parser.module);
  }
  wb200_status st = plan_addresses(program.get());
  if (st != WB200_OK) return st;
  if (backend) {
    DeviceGuard guard(backend->device);
    program->ddr = wb200_spm_image{backend, kDdrBase, program->ddr_bytes, nullptr};
    WB200_CUDA_CHECK(cudaMalloc(&program->ddr.device, program->ddr_bytes));
    WB200_CUDA_CHECK(cudaMemset(program->ddr.device, 0, program->ddr_bytes));
    program->spm.assign(tile_count, wb200_spm_image{backend, 0, program->spm_bytes, nullptr});
    for (uint32_t t = 0; t < tile_count; ++t) {
      // the second half of each allocation is the Tile's private staging area for in-place gather / scatter
      cudaError_t err = cudaMalloc(&program->spm[t].device, 2 * program->spm_bytes);
      if (err == cudaSuccess) err = cudaMemset(program->spm[t].device, 0, 2 * program->spm_bytes);
      cudaStream_t tile_stream = nullptr;
      if (err == cudaSuccess) err = cudaStreamCreateWithFlags(&tile_stream, cudaStreamNonBlocking);
      if (err == cudaSuccess) program->tile_streams.push_back(tile_stream);
      if (err != cudaSuccess) {
        wb200_status failed = fail(WB200_ERR_CUDA, std::string("scratch-pad images: ") + cudaGetErrorString(err));
        wb200_tile_program_destroy(program.release());
        return failed;
      }
    }
    WB200_CUDA_CHECK(cudaEventCreate(&program->begin));
    WB200_CUDA_CHECK(cudaEventCreate(&program->end));
    WB200_CUDA_CHECK(cudaMalloc(&program->numeric_words, 16));
  }
  *out = program.release();
  return WB200_OK;
}

void wb200_tile_program_destroy(wb200_tile_program *program) {
  if (!program) return;
  if (program->backend) {
    DeviceGuard guard(program->backend->device);
    cudaStreamSynchronize(program->backend->stream);
    if (program->ddr.device) cudaFree(program->ddr.device);
    if (program->numeric_words) cudaFree(program->numeric_words);
    for (wb200_spm_image &image : program->spm)
      if (image.device) cudaFree(image.device);
    if (program->begin) cudaEventDestroy(program->begin);
    if (program->end) cudaEventDestroy(program->end);
    for (cudaGraphExec_t graph : program->graph)
      if (graph) cudaGraphExecDestroy(graph);
    for (uint8_t *staging : program->gemm_staging)
      if (staging) cudaFree(staging);
    for (cudaStream_t tile_stream : program->tile_streams) cudaStreamDestroy(tile_stream);
    for (cudaEvent_t event : program->edge_events) cudaEventDestroy(event);
  }
  delete program;
}

wb200_status wb200_tile_program_tensor_count(const wb200_tile_program *program, uint32_t *inputs, uint32_t *outputs) {
  if (!program || !inputs || !outputs) return fail(WB200_ERR_INVALID_ARGUMENT, "null argument");
  *inputs = static_cast<uint32_t>(program->inputs.size());
  *outputs = static_cast<uint32_t>(program->outputs.size());
  return WB200_OK;
}

wb200_status wb200_tile_program_tensor_info(const wb200_tile_program *program, uint32_t is_output, uint32_t index, wb200_tensor_desc *desc,
                                            uint64_t *compact_bytes) {
  if (!program || !desc || !compact_bytes) return fail(WB200_ERR_INVALID_ARGUMENT, "null argument");
  const std::vector<ExternalTensor> &list = is_output ? program->outputs : program->inputs;
  if (index >= list.size()) return fail(WB200_ERR_INVALID_ARGUMENT, "external tensor index out of range");
  *desc = list[index].desc;
  *compact_bytes = list[index].compact_bytes;
  return WB200_OK;
}

wb200_status wb200_tile_program_placement(const wb200_tile_program *program, uint32_t is_output, uint32_t index, uint64_t *address,
                                          uint64_t *physical_bytes, uint64_t *ddr_base, uint64_t *ddr_bytes) {
  if (!program || !address || !physical_bytes || !ddr_base || !ddr_bytes) return fail(WB200_ERR_INVALID_ARGUMENT, "null argument");
  const std::vector<ExternalTensor> &list = is_output ? program->outputs : program->inputs;
  if (index >= list.size()) return fail(WB200_ERR_INVALID_ARGUMENT, "external tensor index out of range");
  *address = list[index].address;
  *physical_bytes = list[index].physical_bytes;
  *ddr_base = kDdrBase;
  *ddr_bytes = program->ddr_bytes;
  return WB200_OK;
}

wb200_status wb200_tile_program_trace(wb200_tile_program *program, wb200_program_command *records, uint64_t capacity, uint64_t *count,
                                      wb200_program_stats *stats) {
  if (!program || !count) return fail(WB200_ERR_INVALID_ARGUMENT, "null argument");
  std::vector<wb200_program_command> trace;
  program->execute = false;
  program->trace = &trace;
  wb200_status st = run_all_tiles(program);
  program->trace = nullptr;
  if (st != WB200_OK) return st;
  *count = trace.size();
  if (stats) *stats = program->stats;
  if (records) {
    if (capacity < trace.size()) return fail(WB200_ERR_LIMIT, "trace buffer smaller than the command count");
    memcpy(records, trace.data(), trace.size() * sizeof(wb200_program_command));
  }
  return WB200_OK;
}

wb200_status wb200_tile_program_run(wb200_tile_program *program, const void *const *inputs, void *const *outputs, uint32_t gemm_policy,
                                    wb200_program_stats *stats) {
  if (!program || !inputs || !outputs) return fail(WB200_ERR_INVALID_ARGUMENT, "null argument");
  if (!program->backend) return fail(WB200_ERR_NO_DEVICE, "the Tile program was loaded without a backend");
  if (gemm_policy > WB200_GEMM_TENSOR) return fail(WB200_ERR_INVALID_ARGUMENT, "unknown GEMM policy");
  wb200_backend *backend = program->backend;
  DeviceGuard guard(backend->device);
  cudaStream_t stream = backend->stream;
  wb200_status st;
  for (size_t i = 0; i < program->inputs.size(); ++i) {
    const ExternalTensor &tensor = program->inputs[i];
    if (!inputs[i]) return fail(WB200_ERR_INVALID_ARGUMENT, "null input tensor");
    uint8_t *storage = program->ddr.device + (tensor.address - kDdrBase);
    if (tensor.desc.layout == WB200_LAYOUT_TENSOR || tensor.desc.layout == WB200_LAYOUT_NTENSOR) {
      WB200_CUDA_CHECK(cudaMemcpyAsync(storage, inputs[i], tensor.compact_bytes, cudaMemcpyHostToDevice, stream));
    } else {
      void *compact;
      if ((st = backend->buffer(10, tensor.compact_bytes, &compact)) != WB200_OK) return st;
      WB200_CUDA_CHECK(cudaMemcpyAsync(compact, inputs[i], tensor.compact_bytes, cudaMemcpyHostToDevice, stream));
      WB200_CUDA_CHECK(cudaMemsetAsync(storage, 0, tensor.physical_bytes, stream));
      if ((st = launch_pack(static_cast<const uint8_t *>(compact), storage, tensor.map, static_cast<int>(tensor.geometry.element_bytes), stream)) != WB200_OK) return st;
      backend->launches += 1;
      WB200_CUDA_CHECK(cudaStreamSynchronize(stream));   // the staging slot is reused by the next tensor
    }
  }
  program->execute = true;
  program->gemm_policy = gemm_policy;
  program->trace = nullptr;
  // Both GEMM policies replay concurrently (one stream per Tile inside a captured graph, one graph per policy); the
  // tensor-core path stages its compact operands in areas private to each Tile. WB200_REPLAY_GRAPH=0 forces the single
  // stream, where the backend's shared slots serve.
  static const bool graph_enabled = [] { const char *env = getenv("WB200_REPLAY_GRAPH"); return !(env && env[0] == '0'); }();
  const bool concurrent = graph_enabled && !program->tile_streams.empty();
  if (concurrent && !program->graph[gemm_policy] && (st = capture_invocation(program)) != WB200_OK) return st;
  WB200_CUDA_CHECK(cudaMemsetAsync(program->numeric_words, 0, 8, stream));
  WB200_CUDA_CHECK(cudaMemsetAsync(program->numeric_words + 2, 0xff, 8, stream));
  WB200_CUDA_CHECK(cudaEventRecord(program->begin, stream));
  if (concurrent) {
    WB200_CUDA_CHECK(cudaGraphLaunch(program->graph[gemm_policy], stream));
    program->stats = program->graph_stats[gemm_policy];
    backend->launches += program->stats.gpu_launches;
  } else {
    for (wb200_spm_image &image : program->spm) { image.stream = nullptr; image.staging = nullptr; image.gemm_staging = nullptr; }
    st = run_all_tiles(program);
    if (st != WB200_OK) { cudaStreamSynchronize(stream); return st; }
  }
  WB200_CUDA_CHECK(cudaEventRecord(program->end, stream));
  if ((st = read_device_status(backend, stream, nullptr)) != WB200_OK) return st;
  float elapsed = 0.f;
  WB200_CUDA_CHECK(cudaEventElapsedTime(&elapsed, program->begin, program->end));
  program->stats.device_ms = elapsed;
  uint32_t numeric[4] = {0, 0, 0, 0};
  WB200_CUDA_CHECK(cudaMemcpyAsync(numeric, program->numeric_words, sizeof(numeric), cudaMemcpyDeviceToHost, stream));
  WB200_CUDA_CHECK(cudaStreamSynchronize(stream));
  unsigned long long refused;
  memcpy(&refused, numeric + 2, sizeof(refused));
  if (refused != ~0ull) {   // a failed command fails the invocation; outputs are not returned
    if ((refused & 0xff) == 4) return fail(WB200_ERR_UNSUPPORTED, "MaskMove requires canonical zero/one mask values at element " + std::to_string(refused >> 8));
    return convert_refusal(refused);
  }
  program->stats.numeric_flags = numeric[0];
  for (size_t i = 0; i < program->outputs.size(); ++i) {
    const ExternalTensor &tensor = program->outputs[i];
    if (!outputs[i]) return fail(WB200_ERR_INVALID_ARGUMENT, "null output tensor");
    const uint8_t *storage = program->ddr.device + (tensor.address - kDdrBase);
    if (tensor.desc.layout == WB200_LAYOUT_TENSOR || tensor.desc.layout == WB200_LAYOUT_NTENSOR) {
      WB200_CUDA_CHECK(cudaMemcpyAsync(outputs[i], storage, tensor.compact_bytes, cudaMemcpyDeviceToHost, stream));
    } else {
      void *compact;
      if ((st = backend->buffer(10, tensor.compact_bytes, &compact)) != WB200_OK) return st;
      if ((st = launch_unpack(storage, static_cast<uint8_t *>(compact), tensor.map, static_cast<int>(tensor.geometry.element_bytes), stream)) != WB200_OK) return st;
      backend->launches += 1;
      WB200_CUDA_CHECK(cudaMemcpyAsync(outputs[i], compact, tensor.compact_bytes, cudaMemcpyDeviceToHost, stream));
    }
    WB200_CUDA_CHECK(cudaStreamSynchronize(stream));
  }
  if (stats) *stats = program->stats;
  return WB200_OK;
}

// ------------------------------------------------------------------ command-level movement entry points
static wb200_status movement_args(const uint32_t strides[3], const uint32_t iterations[3], uint32_t inner_bytes, uint32_t byte_count, StridedLayout *layout) {
  if (!strides || !iterations) return fail(WB200_ERR_INVALID_ARGUMENT, "null argument");
  layout->inner_bytes = inner_bytes;
  for (int d = 0; d < 3; ++d) { layout->strides[d] = strides[d]; layout->iterations[d] = iterations[d]; }
  return check_layout(*layout, byte_count);
}

wb200_status wb200_target_call_rdma(wb200_spm_image *ddr, wb200_spm_image *spm, uint64_t source, uint64_t destination, uint32_t byte_count,
                                    uint32_t inner_bytes, const uint32_t strides[3], const uint32_t iterations[3]) {
  if (!ddr || !spm || ddr->backend != spm->backend) return fail(WB200_ERR_INVALID_ARGUMENT, "images must belong to one backend");
  StridedLayout strided;
  wb200_status st = movement_args(strides, iterations, inner_bytes, byte_count, &strided);
  if (st != WB200_OK) return st;
  DeviceGuard guard(spm->backend->device);
  uint64_t launches = 0;
  st = enqueue_image_copy(ddr, source, strided, spm, destination, contiguous_layout(inner_bytes, strided_segments(strided)), true, &launches);
  if (st != WB200_OK) return st;
  return read_device_status(spm->backend, spm->backend->stream, nullptr);
}

wb200_status wb200_target_call_wdma(wb200_spm_image *spm, wb200_spm_image *ddr, uint64_t source, uint64_t destination, uint32_t byte_count,
                                    uint32_t inner_bytes, const uint32_t strides[3], const uint32_t iterations[3]) {
  if (!ddr || !spm || ddr->backend != spm->backend) return fail(WB200_ERR_INVALID_ARGUMENT, "images must belong to one backend");
  StridedLayout strided;
  wb200_status st = movement_args(strides, iterations, inner_bytes, byte_count, &strided);
  if (st != WB200_OK) return st;
  DeviceGuard guard(spm->backend->device);
  uint64_t launches = 0;
  st = enqueue_image_copy(spm, source, contiguous_layout(inner_bytes, strided_segments(strided)), ddr, destination, strided, true, &launches);
  if (st != WB200_OK) return st;
  return read_device_status(spm->backend, spm->backend->stream, nullptr);
}

wb200_status wb200_target_call_gather_scatter(wb200_spm_image *spm, uint64_t source, uint64_t destination, uint32_t byte_count,
                                              uint32_t inner_bytes, const uint32_t source_strides[3], const uint32_t source_iterations[3],
                                              const uint32_t destination_strides[3], const uint32_t destination_iterations[3]) {
  if (!spm) return fail(WB200_ERR_INVALID_ARGUMENT, "null argument");
  StridedLayout from, to;
  wb200_status st;
  if ((st = movement_args(source_strides, source_iterations, inner_bytes, byte_count, &from)) != WB200_OK) return st;
  if ((st = movement_args(destination_strides, destination_iterations, inner_bytes, byte_count, &to)) != WB200_OK) return st;
  DeviceGuard guard(spm->backend->device);
  uint64_t launches = 0;
  if ((st = enqueue_image_copy(spm, source, from, spm, destination, to, true, &launches)) != WB200_OK) return st;
  return read_device_status(spm->backend, spm->backend->stream, nullptr);
}

wb200_status wb200_target_call_memset(wb200_spm_image *spm, uint64_t destination, uint32_t value_bits, uint32_t element_count, uint32_t format) {
  if (!spm) return fail(WB200_ERR_INVALID_ARGUMENT, "null argument");
  DeviceGuard guard(spm->backend->device);
  uint64_t launches = 0;
  wb200_status st = enqueue_image_fill(spm, destination, value_bits, element_count, format, true, &launches);
  if (st != WB200_OK) return st;
  return read_device_status(spm->backend, spm->backend->stream, nullptr);
}

wb200_status wb200_target_call_bit2fp(wb200_spm_image *spm, uint64_t source, uint64_t destination, uint32_t element_count, uint32_t format) {
  if (!spm) return fail(WB200_ERR_INVALID_ARGUMENT, "null argument");
  DeviceGuard guard(spm->backend->device);
  uint64_t launches = 0;
  wb200_status st = enqueue_image_bit2fp(spm, source, destination, element_count, format, true, &launches);
  if (st != WB200_OK) return st;
  return read_device_status(spm->backend, spm->backend->stream, nullptr);
}

wb200_status wb200_target_call_mask_move(wb200_spm_image *spm, uint64_t source, uint64_t mask, uint64_t destination, uint32_t element_count,
                                         uint32_t format) {
  if (!spm) return fail(WB200_ERR_INVALID_ARGUMENT, "null argument");
  wb200_backend *backend = spm->backend;
  DeviceGuard guard(backend->device);
  void *word;
  wb200_status st = backend->buffer(3, sizeof(unsigned long long), &word);
  if (st != WB200_OK) return st;
  cudaStream_t stream = spm->work_stream();
  uint64_t launches = 0;
  WB200_CUDA_CHECK(cudaMemsetAsync(word, 0xff, sizeof(unsigned long long), stream));
  // validate first: a refused mask value leaves the destination untouched
  if ((st = enqueue_image_mask_move(spm, source, mask, destination, element_count, format, true, 0, static_cast<unsigned long long *>(word), &launches)) != WB200_OK) return st;
  unsigned long long refused = ~0ull;
  WB200_CUDA_CHECK(cudaMemcpyAsync(&refused, word, sizeof(refused), cudaMemcpyDeviceToHost, stream));
  WB200_CUDA_CHECK(cudaStreamSynchronize(stream));
  if (refused != ~0ull)
    return fail(WB200_ERR_UNSUPPORTED, "MaskMove requires canonical zero/one mask values at element " + std::to_string(refused >> 8));
  if ((st = enqueue_image_mask_move(spm, source, mask, destination, element_count, format, true, 1, static_cast<unsigned long long *>(word), &launches)) != WB200_OK) return st;
  return read_device_status(backend, backend->stream, nullptr);
}

}  // extern "C"
