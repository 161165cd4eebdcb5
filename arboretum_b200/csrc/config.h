// Training configuration: the nested JSON document of the reference
// (src/core/param.h:20-79, src/core/json_conversion.h:51-167) with the same key
// names and defaults.  Unknown keys are ignored, like in the reference (so the
// `gamma` key that its tests pass has no effect here either).
#pragma once
#include <string>

#include "json.h"

namespace arb {

enum Objective {  // param.h:7-14
  kLinearRegression = 0,
  kLogisticRegression = 1,
  kSoftMaxOneVsAll = 3,
};
enum Method { kExact = 0, kHist = 1 };  // param.h:16

struct TreeParam {  // param.h:20-43 (defaults :21-27)
  unsigned depth = 8;  // = max_depth + 1 (json_conversion.h:108-112)
  float min_child_weight = 1.0f;
  unsigned min_leaf_size = 1;
  float colsample_bytree = 1.0f;
  float colsample_bylevel = 1.0f;
  float gamma_absolute = 0.0f;
  float gamma_relative = 0.0f;
  float lambda = 1.0f;
  float alpha = 0.0f;
  float initial_y = 0.5f;
  float eta = 0.3f;
  float max_leaf_weight = 0.0f;
  float scale_pos_weight = 1.0f;
  unsigned labels_count = 1;
};

struct Verbose {  // param.h:45-50
  bool gpu = false, booster = false, data = false;
};

struct Internals {  // param.h:52-62 (defaults :54-57)
  bool double_precision = false;  // accepted; sums here are always exact integers
  unsigned compute_overlap = 2;   // accepted; the level loop here is one stream
  unsigned seed = 0;
  bool use_hist_subtraction_trick = true;
  bool upload_features = true;
  int hist_size = 255;
  // additive keys of this build
  int quant_bits = 0;    // fixed-point bits of a gradient (see hist.cu); 0 = by the row count
  int device = -1;       // CUDA device ordinal, -1 = current device
  bool missing_bin = true;  // NaN -> dedicated bin id hist_size (always right)
  long long chunk_rows = 0;  // out-of-core: rows per streamed chunk, 0 = in-core
  int resident_chunks = -1;  // out-of-core: chunks kept in HBM (-1 = as many as fit)
};

struct Configuration {
  int method = kHist;
  int objective = -1;
  TreeParam tree;
  Verbose verbose;
  Internals internal;

  static int parse_objective(const Json &j) {
    if (j.type == Json::Str) {
      if (j.str == "reg:linear") return kLinearRegression;
      if (j.str == "reg:logistic") return kLogisticRegression;
      if (j.str == "multi:softmax") return kSoftMaxOneVsAll;
      throw std::runtime_error("Unknown objective function " + j.str);
    }
    return int(j.as_num());
  }
  static int parse_method(const Json &j) {
    if (j.type == Json::Str) {
      if (j.str == "hist") return kHist;
      if (j.str == "exact") return kExact;
      throw std::runtime_error("Unknown method " + j.str);
    }
    return int(j.as_num());
  }

  static Configuration Parse(const char *text) {  // param.cpp:47-51
    Configuration c;
    const Json j = JsonParser(text).parse();
    if (j.type != Json::Obj) throw std::runtime_error("configuration must be a JSON object");
    if (j.has("method")) c.method = parse_method(j.at("method"));
    if (j.has("objective")) c.objective = parse_objective(j.at("objective"));
    if (j.has("tree")) {
      const Json &t = j.at("tree");
#define ARB_GET(field, key, T) \
  if (t.has(key)) c.tree.field = T(t.at(key).as_num())
      if (t.has("max_depth")) c.tree.depth = unsigned(int(t.at("max_depth").as_num()) + 1);
      ARB_GET(min_child_weight, "min_child_weight", float);
      ARB_GET(min_leaf_size, "min_leaf_size", unsigned);
      ARB_GET(colsample_bytree, "colsample_bytree", float);
      ARB_GET(colsample_bylevel, "colsample_bylevel", float);
      ARB_GET(gamma_absolute, "gamma_absolute", float);
      ARB_GET(gamma_relative, "gamma_relative", float);
      ARB_GET(lambda, "lambda", float);
      ARB_GET(alpha, "alpha", float);
      ARB_GET(initial_y, "initial_y", float);
      ARB_GET(eta, "eta", float);
      ARB_GET(max_leaf_weight, "max_leaf_weight", float);
      ARB_GET(scale_pos_weight, "scale_pos_weight", float);
      ARB_GET(labels_count, "labels_count", unsigned);
#undef ARB_GET
    }
    if (j.has("verbose")) {
      const Json &v = j.at("verbose");
      if (v.has("gpu")) c.verbose.gpu = v.at("gpu").as_bool();
      if (v.has("booster")) c.verbose.booster = v.at("booster").as_bool();
      if (v.has("data")) c.verbose.data = v.at("data").as_bool();
    }
    if (j.has("internals")) {
      const Json &i = j.at("internals");
      if (i.has("double_precision")) c.internal.double_precision = i.at("double_precision").as_bool();
      if (i.has("compute_overlap")) c.internal.compute_overlap = unsigned(i.at("compute_overlap").as_num());
      if (i.has("seed")) c.internal.seed = unsigned(i.at("seed").as_num());
      if (i.has("use_hist_subtraction_trick"))
        c.internal.use_hist_subtraction_trick = i.at("use_hist_subtraction_trick").as_bool();
      if (i.has("upload_features")) c.internal.upload_features = i.at("upload_features").as_bool();
      if (i.has("hist_size")) c.internal.hist_size = int(i.at("hist_size").as_num());
      if (i.has("quant_bits")) c.internal.quant_bits = int(i.at("quant_bits").as_num());
      if (i.has("device")) c.internal.device = int(i.at("device").as_num());
      if (i.has("missing_bin")) c.internal.missing_bin = i.at("missing_bin").as_bool();
      if (i.has("chunk_rows")) c.internal.chunk_rows = (long long)i.at("chunk_rows").as_num();
      if (i.has("resident_chunks")) c.internal.resident_chunks = int(i.at("resident_chunks").as_num());
    }
    return c;
  }

  Json ToJson() const {  // json_conversion.h:51-155: the keys the reference dumps
    Json j = Json::object();
    j["method"] = Json::integer(method);
    j["objective"] = Json::integer(objective);
    Json t = Json::object();
    t["max_depth"] = Json::integer((long long)tree.depth - 1);
    t["min_child_weight"] = Json::number(tree.min_child_weight);
    t["min_leaf_size"] = Json::integer(tree.min_leaf_size);
    t["colsample_bytree"] = Json::number(tree.colsample_bytree);
    t["colsample_bylevel"] = Json::number(tree.colsample_bylevel);
    t["gamma_absolute"] = Json::number(tree.gamma_absolute);
    t["gamma_relative"] = Json::number(tree.gamma_relative);
    t["lambda"] = Json::number(tree.lambda);
    t["alpha"] = Json::number(tree.alpha);
    t["initial_y"] = Json::number(tree.initial_y);
    t["eta"] = Json::number(tree.eta);
    t["max_leaf_weight"] = Json::number(tree.max_leaf_weight);
    t["scale_pos_weight"] = Json::number(tree.scale_pos_weight);
    t["labels_count"] = Json::integer(tree.labels_count);
    j["tree"] = t;
    Json v = Json::object();
    v["gpu"] = Json::boolean(verbose.gpu);
    v["booster"] = Json::boolean(verbose.booster);
    v["data"] = Json::boolean(verbose.data);
    j["verbose"] = v;
    Json i = Json::object();
    i["double_precision"] = Json::boolean(internal.double_precision);
    i["compute_overlap"] = Json::integer(internal.compute_overlap);
    i["seed"] = Json::integer(internal.seed);
    i["use_hist_subtraction_trick"] = Json::boolean(internal.use_hist_subtraction_trick);
    i["upload_features"] = Json::boolean(internal.upload_features);
    i["hist_size"] = Json::integer(internal.hist_size);
    j["internals"] = i;
    return j;
  }
};

}  // namespace arb
