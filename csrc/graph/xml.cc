// Minimal XML tree for the topology dump (MCCL_TOPO_DUMP_FILE) and its round trip.
#include <cstdio>
#include <cstring>

#include "graph.h"

namespace mccl {

XmlNode::~XmlNode() { for (XmlNode* s : subs) delete s; }

XmlNode* xmlAddNode(XmlNode* parent, const char* name) {
  XmlNode* n = new XmlNode();
  n->name = name;
  if (parent) parent->subs.push_back(n);
  return n;
}

void xmlSetAttr(XmlNode* n, const char* key, const std::string& value) {
  for (auto& kv : n->attrs) if (kv.first == key) { kv.second = value; return; }
  n->attrs.emplace_back(key, value);
}
void xmlSetAttrInt(XmlNode* n, const char* key, long long v) { xmlSetAttr(n, key, std::to_string(v)); }
void xmlSetAttrFloat(XmlNode* n, const char* key, double v) {
  char buf[64];
  snprintf(buf, sizeof(buf), "%.6g", v);
  xmlSetAttr(n, key, buf);
}
const char* xmlGetAttr(const XmlNode* n, const char* key) {
  for (auto& kv : n->attrs) if (kv.first == key) return kv.second.c_str();
  return nullptr;
}

static std::string escape(const std::string& s) {
  std::string o;
  for (char c : s) {
    switch (c) {
      case '&': o += "&amp;"; break;
      case '<': o += "&lt;"; break;
      case '>': o += "&gt;"; break;
      case '"': o += "&quot;"; break;
      default: o += c;
    }
  }
  return o;
}
static std::string unescape(const std::string& s) {
  std::string o;
  for (size_t i = 0; i < s.size(); ++i) {
    if (s[i] != '&') { o += s[i]; continue; }
    if (!s.compare(i, 5, "&amp;")) { o += '&'; i += 4; }
    else if (!s.compare(i, 4, "&lt;")) { o += '<'; i += 3; }
    else if (!s.compare(i, 4, "&gt;")) { o += '>'; i += 3; }
    else if (!s.compare(i, 6, "&quot;")) { o += '"'; i += 5; }
    else o += s[i];
  }
  return o;
}

static void emit(const XmlNode* n, int depth, std::string* out) {
  out->append(depth * 2, ' ');
  *out += "<" + n->name;
  for (auto& kv : n->attrs) *out += " " + kv.first + "=\"" + escape(kv.second) + "\"";
  if (n->subs.empty()) { *out += "/>\n"; return; }
  *out += ">\n";
  for (const XmlNode* s : n->subs) emit(s, depth + 1, out);
  out->append(depth * 2, ' ');
  *out += "</" + n->name + ">\n";
}

std::string xmlToString(const XmlNode* root) {
  std::string out;
  if (root) emit(root, 0, &out);
  return out;
}

namespace {
struct Parser {
  const std::string& t;
  size_t i = 0;
  explicit Parser(const std::string& text) : t(text) {}
  void ws() { while (i < t.size() && strchr(" \t\r\n", t[i])) ++i; }
  std::string ident() {
    size_t s = i;
    while (i < t.size() && !strchr(" \t\r\n=/>\"", t[i])) ++i;
    return t.substr(s, i - s);
  }
  XmlNode* element() {
    ws();
    if (i >= t.size() || t[i] != '<') return nullptr;
    ++i;
    XmlNode* n = new XmlNode();
    n->name = ident();
    for (;;) {
      ws();
      if (i >= t.size()) { delete n; return nullptr; }
      if (t[i] == '/') { i += 2; return n; }          // "/>"
      if (t[i] == '>') { ++i; break; }
      std::string key = ident();
      ws();
      if (i >= t.size() || t[i] != '=') { delete n; return nullptr; }
      ++i; ws();
      if (i >= t.size() || t[i] != '"') { delete n; return nullptr; }
      size_t e = t.find('"', i + 1);
      if (e == std::string::npos) { delete n; return nullptr; }
      n->attrs.emplace_back(key, unescape(t.substr(i + 1, e - i - 1)));
      i = e + 1;
    }
    for (;;) {
      ws();
      if (i + 1 < t.size() && t[i] == '<' && t[i + 1] == '/') {
        size_t e = t.find('>', i);
        i = (e == std::string::npos) ? t.size() : e + 1;
        return n;
      }
      XmlNode* c = element();
      if (c == nullptr) { delete n; return nullptr; }
      n->subs.push_back(c);
    }
  }
};
}  // namespace

XmlNode* xmlParse(const std::string& text) { Parser p(text); return p.element(); }

XmlNode* topoToXml(const TopoSystem& sys, const TopoGraph* graphs, int nGraphs, const TunerModel* tuner) {
  XmlNode* root = xmlAddNode(nullptr, "system");
  xmlSetAttrInt(root, "version", MCCL_VERSION_CODE);
  xmlSetAttrInt(root, "ranks", (long long)sys.nodes.size());
  xmlSetAttrInt(root, "nvls", sys.nvls);
  xmlSetAttrInt(root, "netAllToAll", sys.netAllToAll);
  for (const TopoNode& nd : sys.nodes) {
    XmlNode* g = xmlAddNode(root, nd.device >= 0 ? "gpu" : "host");
    xmlSetAttrInt(g, "rank", nd.rank);
    xmlSetAttrInt(g, "dev", nd.device);
    xmlSetAttrInt(g, "sm", nd.smCount);
    xmlSetAttrInt(g, "cc", nd.cc);
    xmlSetAttrInt(g, "hbmGiB", (long long)nd.hbmGiB);
    xmlSetAttrInt(g, "multicast", nd.multicast);
    xmlSetAttr(g, "busid", nd.busId);
    char hh[32];
    snprintf(hh, sizeof(hh), "%016llx", (unsigned long long)nd.hostHash);
    xmlSetAttr(g, "host", hh);
    for (const TopoLink& l : nd.links) {
      XmlNode* x = xmlAddNode(g, "link");
      xmlSetAttrInt(x, "peer", l.remote);
      xmlSetAttr(x, "type", linkTypeStr(l.type));
      xmlSetAttrFloat(x, "bw", l.bw);
      if (l.measured > 0.f) xmlSetAttrFloat(x, "measured", l.measured);
      if (l.latencyUs > 0.f) xmlSetAttrFloat(x, "latency_us", l.latencyUs);
    }
  }
  for (int i = 0; i < nGraphs && graphs; ++i) {
    XmlNode* a = xmlAddNode(root, "algo");
    xmlSetAttr(a, "name", mcclAlgoStr(graphs[i].algo));
    xmlSetAttrInt(a, "viable", graphs[i].viable);
    xmlSetAttrFloat(a, "bw", graphs[i].bw);
    xmlSetAttrInt(a, "channels", graphs[i].nChannels);
    std::string order;
    for (size_t k = 0; k < graphs[i].order.size(); ++k) order += (k ? "," : "") + std::to_string(graphs[i].order[k]);
    xmlSetAttr(a, "order", order);
    if (tuner) {
      xmlSetAttrFloat(a, "alpha_us", tuner->alphaUs[graphs[i].algo]);
      xmlSetAttrFloat(a, "step_us", tuner->stepUs[graphs[i].algo]);
      xmlSetAttrFloat(a, "model_bw", tuner->bw[graphs[i].algo]);
    }
  }
  return root;
}

mcclResult_t topoDumpXmlToFile(const TopoSystem& sys, const TopoGraph* graphs, int nGraphs, const TunerModel* tuner, const char* path) {
  XmlNode* root = topoToXml(sys, graphs, nGraphs, tuner);
  std::string s = xmlToString(root);
  delete root;
  FILE* f = fopen(path, "w");
  if (f == nullptr) MCCLFAIL(mcclSystemError);
  fwrite(s.data(), 1, s.size(), f);
  fclose(f);
  return mcclSuccess;
}

static const char* fuseKey(const XmlNode* n) {
  const char* k = xmlGetAttr(n, "rank");
  if (k == nullptr) k = xmlGetAttr(n, "peer");
  if (k == nullptr) k = xmlGetAttr(n, "name");
  return k;
}

void xmlFuse(XmlNode* dst, const XmlNode* src) {
  for (auto& kv : src->attrs) if (xmlGetAttr(dst, kv.first.c_str()) == nullptr) xmlSetAttr(dst, kv.first.c_str(), kv.second);
  for (const XmlNode* s : src->subs) {
    XmlNode* match = nullptr;
    const char* sk = fuseKey(s);
    for (XmlNode* d : dst->subs) {
      const char* dk = fuseKey(d);
      if (d->name == s->name && sk && dk && !strcmp(sk, dk)) { match = d; break; }
    }
    if (match == nullptr) match = xmlAddNode(dst, s->name.c_str());
    xmlFuse(match, s);
  }
}

}  // namespace mccl
